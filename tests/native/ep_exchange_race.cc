// The expert-parallel token exchange over peer memory (parallel/nvlink_ep.py, csrc/ep.cu), executed by CPU threads (one
// per rank: all of its kernels run on one in-order stream) on plain arrays. Built with -fsanitize=thread.
//
// One dispatch + combine call c (parity p = c % 2, version v = calls made on that parity):
//   publish  : write my per-expert counts into row `me` of every rank's table[p] (peer stores); flags[p][me] on every
//              rank = v (release)
//   maps     : wait my flags[p][r] >= v for all r (acquire); read my table[p]; every rank derives the same slots: the
//              rows rank s sends to expert e start at base(e) + sum of the counts of ranks before s
//   push     : store each of my rows into its slot of the owner's recv[p] (peer stores); add 1 to every rank's
//              arrive_fwd[p] (release)
//   wait     : my arrive_fwd[p] >= v * world (acquire); copy my recv[p] out (plain loads)
//   combine  : the same the other way: rows go back to their sources' ret[p], arrive_rev[p], wait, copy out
// Nothing else orders ranks. Tables, flags, buffers and counters exist twice, used by alternating calls (as in the
// runtime, where forward and backward exchanges of neighbouring layers interleave); in this forward-only sequence every
// call ends with a full exchange, so one set would do as well (-DSINGLE_BUFFER, also race-free).
// -DDROP_ARRIVE_WAIT copies the receive buffer out without waiting for the arrival counter: ThreadSanitizer then reports
// the peers' row stores against the copy-out. The test runs the shipped protocol and this negative control.
#include <stdio.h>

#include <thread>
#include <vector>

#include "protocol.h"

namespace {

constexpr int kWorld = 4, kExperts = 8, kLocal = kExperts / kWorld, kRows = 24, kDim = 4, kCalls = 12;
constexpr int kCap = kWorld * kRows;
constexpr uint64_t kPollLimit = 1ull << 34;
#ifdef SINGLE_BUFFER
constexpr int kSets = 1;
#else
constexpr int kSets = 2;
#endif

struct Rank {
  int table[kSets][kWorld * kExperts];
  float recv[kSets][kCap * kDim];
  float ret[kSets][kRows * kDim];
  alignas(64) int flags[kSets][kWorld];
  alignas(64) int arrive_fwd[kSets];
  alignas(64) int arrive_rev[kSets];
  double checksum;
};
Rank g_rank[kWorld];
int g_failed = 0;

bool wait_ge(const int* f, int expected) {
  int seen;
  if (tt::proto::wait_flag_ge(f, expected, 0, kPollLimit, &seen)) return true;
  __atomic_store_n(&g_failed, 1, __ATOMIC_RELAXED);
  return false;
}

// rank s sends count(s, e, c) rows to expert e in call c; every rank's rows add up to kRows
int count(int s, int e, int c) {
  const int hot = (s + c) % kExperts;                 // a shifting hot expert
  return e == hot ? kRows - 2 * (kExperts - 1) : 2;
}

void run_rank(int me) {
  Rank& R = g_rank[me];
  for (int c = 1; c <= kCalls; ++c) {
    const int p = c % kSets;
    const int v = kSets == 2 ? (c % 2 ? (c + 1) / 2 : c / 2) : c;
    // ---- publish my counts
    for (int d = 0; d < kWorld; ++d) {
      for (int e = 0; e < kExperts; ++e) g_rank[d].table[p][me * kExperts + e] = count(me, e, c);
    }
    for (int d = 0; d < kWorld; ++d) tt::proto::st_release_sys(&g_rank[d].flags[p][me], v);
    // ---- maps
    for (int r = 0; r < kWorld; ++r)
      if (!wait_ge(&R.flags[p][r], v)) return;
    int start[kExperts];                               // slot on the owner where my rows of expert e begin
    for (int d = 0; d < kWorld; ++d) {
      int base = 0;
      for (int el = 0; el < kLocal; ++el) {
        const int e = d * kLocal + el;
        int total = 0, before = 0;
        for (int s = 0; s < kWorld; ++s) {
          const int n = R.table[p][s * kExperts + e];
          if (s < me) before += n;
          total += n;
        }
        start[e] = base + before;
        base += total;
      }
    }
    // ---- push my rows (sorted by expert) to their owners
    int j = 0;
    for (int e = 0; e < kExperts; ++e) {
      const int owner = e / kLocal;
      for (int i = 0; i < R.table[p][me * kExperts + e]; ++i, ++j)
        for (int k = 0; k < kDim; ++k) g_rank[owner].recv[p][(start[e] + i) * kDim + k] = 1000.f * me + j + 0.1f * k + c;
    }
    for (int d = 0; d < kWorld; ++d) __atomic_fetch_add(&g_rank[d].arrive_fwd[p], 1, __ATOMIC_RELEASE);
#ifndef DROP_ARRIVE_WAIT
    if (!wait_ge(&R.arrive_fwd[p], v * kWorld)) return;
#endif
    // ---- copy out what I received and send every row back to its source
    int seg = 0;
    for (int el = 0; el < kLocal; ++el) {
      const int e = me * kLocal + el;
      for (int s = 0; s < kWorld; ++s) {
        int src0 = 0;                                  // sorted position on rank s where its rows of expert e begin
        for (int e2 = 0; e2 < e; ++e2) src0 += R.table[p][s * kExperts + e2];
        const int n = R.table[p][s * kExperts + e];
        for (int i = 0; i < n; ++i)
          for (int k = 0; k < kDim; ++k) g_rank[s].ret[p][(src0 + i) * kDim + k] = 2.f * R.recv[p][(seg + i) * kDim + k];
        seg += n;
      }
    }
    for (int d = 0; d < kWorld; ++d) __atomic_fetch_add(&g_rank[d].arrive_rev[p], 1, __ATOMIC_RELEASE);
    if (!wait_ge(&R.arrive_rev[p], v * kWorld)) return;
    for (int i = 0; i < kRows * kDim; ++i) R.checksum += R.ret[p][i];
    if (me == c % kWorld) std::this_thread::yield();   // ranks drift apart by up to one call
  }
}

}  // namespace

int main() {
  std::vector<std::thread> threads;
  for (int r = 0; r < kWorld; ++r) threads.emplace_back(run_rank, r);
  for (auto& t : threads) t.join();
  if (g_failed) {
    fprintf(stderr, "a bounded wait ran out\n");
    return 2;
  }
  // every row came back doubled: rank r sent 1000 r + j + 0.1 k + c for its kRows rows in every call
  double want = 0.0, got = 0.0;
  for (int r = 0; r < kWorld; ++r) {
    got += g_rank[r].checksum;
    for (int c = 1; c <= kCalls; ++c)
      for (int j = 0; j < kRows; ++j)
        for (int k = 0; k < kDim; ++k) want += 2.0 * (1000.0 * r + j + 0.1f * k + c);
  }
  printf("checksum %.3f expected %.3f\n", got, want);
  return (got > want * 0.999999 && got < want * 1.000001) ? 0 : 3;
}
