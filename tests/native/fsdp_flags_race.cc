// The version-flag protocol of the peer-memory FSDP transport, executed by CPU threads (one per rank) on plain arrays.
// Built with -fsanitize=thread: every data access that the flags do not order is reported as a data race.
//
// Per rank two threads stand for its two in-order streams, as in parallel/fsdp.py: the compute stream (optimizer,
// gathers, backward) and the reduce stream (reduce-scatter kernels), joined by local events. Per optimizer step and unit,
// as parallel/nvlink_comm.py issues it:
//   optimizer     : (compute) after the reduce stream has finished the step's reductions: read the gradient shard, write
//                   the shadow shard (plain stores); flag_shadow[me] = V (release)
//   all-gather    : (compute) wait all flag_shadow >= V (acquire); read every peer's shadow shard
//   per micro-batch m and unit u, back to front:
//     guard       : (compute) if this is not the first backward since the optimizer step, wait all flag_done >= G ("my
//                   reduce has read your staging buffer")
//     backward    : (compute) write the whole staging buffer (plain stores); event written[u] = G + 1 for the reduce stream;
//                   go on with the next unit without waiting for the reduction
//     reduce      : (reduce) after written[u]: flag_grad[me] = G + 1 (release); wait all flag_grad >= G + 1; read my slice
//                   of every peer's staging buffer, add into the gradient shard; flag_done[me] = G + 1 (release); event
//                   reduced[u] for the compute stream
// Across optimizer steps nothing waits on flag_done: a peer's next all-gather needs this rank's next flag_shadow, which
// follows (through the reduced[] events) this rank's reduce reads.
//
// -DDROP_STAGING_WAIT leaves the guard out: with two or more micro-batches ThreadSanitizer then reports the race
// between a rank's next backward (staging writes) and a peer's reduce stream still reading. The test runs both builds.
#include <stdio.h>
#include <stdlib.h>

#include <thread>
#include <vector>

#include "protocol.h"

namespace {

constexpr int kWorld = 4, kUnits = 3, kChunk = 64, kSteps = 4, kMicro = 3;
constexpr uint64_t kPollLimit = 1ull << 34;

struct Rank {
  float shadow[kUnits][kChunk];                 // this rank's shard of every unit (peers read it)
  float staging[kUnits][kWorld * kChunk];       // gradients in the gathered layout (owners read their slice)
  float grad[kUnits][kChunk];                   // this rank's reduced gradient shard
  float gathered[kUnits][kWorld * kChunk];      // private
  alignas(64) int flag_shadow[kUnits];
  alignas(64) int flag_grad[kUnits];
  alignas(64) int flag_done[kUnits];
};

Rank g_rank[kWorld];
int g_failed = 0;

bool wait_all(int Rank::*dummy, int unit, int expected, int which) {
  (void)dummy;
  for (int r = 0; r < kWorld; ++r) {
    const int* f = which == 0 ? &g_rank[r].flag_shadow[unit] : which == 1 ? &g_rank[r].flag_grad[unit] : &g_rank[r].flag_done[unit];
    int seen;
    if (!tt::proto::wait_flag_ge(f, expected, 0, kPollLimit, &seen)) {
      __atomic_store_n(&g_failed, 1, __ATOMIC_RELAXED);
      return false;
    }
  }
  return true;
}

struct Local {                                   // events between the two streams of one rank
  alignas(64) int written[kUnits];
  alignas(64) int reduced[kUnits];
};
Local g_local[kWorld];

bool wait_local(const int* ev, int expected) {
  int seen;
  if (tt::proto::wait_flag_ge(ev, expected, 0, kPollLimit, &seen)) return true;
  __atomic_store_n(&g_failed, 1, __ATOMIC_RELAXED);
  return false;
}

void compute_stream(int me) {
  Rank& R = g_rank[me];
  Local& L = g_local[me];
  int grad_version[kUnits] = {0, 0, 0};
  for (int step = 1; step <= kSteps; ++step) {
    // ---- optimizer: after the reduce stream finished the previous step (wait_for_reduce), then new shadow shards
    for (int u = 0; u < kUnits; ++u) {
      if (!wait_local(&L.reduced[u], grad_version[u])) return;
      for (int i = 0; i < kChunk; ++i) R.shadow[u][i] = 0.5f * R.shadow[u][i] - 0.01f * R.grad[u][i] + step + me;
      tt::proto::st_release_sys(&R.flag_shadow[u], step);
    }
    for (int m = 0; m < kMicro; ++m) {
      for (int u = 0; u < kUnits; ++u) {                      // forward: gather front to back
        if (!wait_all(nullptr, u, step, 0)) return;
        for (int r = 0; r < kWorld; ++r)
          for (int i = 0; i < kChunk; ++i) R.gathered[u][r * kChunk + i] = g_rank[r].shadow[u][i];
      }
      for (int u = kUnits - 1; u >= 0; --u) {                 // backward: back to front
#ifndef DROP_STAGING_WAIT
        if (m > 0 && !wait_all(nullptr, u, grad_version[u], 2)) return;      // peers have read the previous staging content
#endif
        for (int i = 0; i < kWorld * kChunk; ++i) R.staging[u][i] = R.gathered[u][i] * 0.001f + m;
        tt::proto::st_release_sys(&L.written[u], ++grad_version[u]);
      }
    }
  }
  for (int u = 0; u < kUnits; ++u) wait_local(&L.reduced[u], grad_version[u]);
}

void reduce_stream(int me) {
  Rank& R = g_rank[me];
  Local& L = g_local[me];
  int g = 0;
  for (int step = 1; step <= kSteps; ++step) {
    for (int m = 0; m < kMicro; ++m) {
      ++g;
      for (int u = kUnits - 1; u >= 0; --u) {
        if (!wait_local(&L.written[u], g)) return;
        tt::proto::st_release_sys(&R.flag_grad[u], g);
        if (!wait_all(nullptr, u, g, 1)) return;
        std::this_thread::yield();                            // a slow reduction: peers run ahead meanwhile
        for (int i = 0; i < kChunk; ++i) {
          float a = 0.f;
          for (int r = 0; r < kWorld; ++r) a += g_rank[r].staging[u][me * kChunk + i];
          R.grad[u][i] = m == 0 ? a : R.grad[u][i] + a;
        }
        tt::proto::st_release_sys(&R.flag_done[u], g);
        tt::proto::st_release_sys(&L.reduced[u], g);
      }
    }
  }
}

}  // namespace

int main() {
  std::vector<std::thread> threads;
  for (int r = 0; r < kWorld; ++r) {
    threads.emplace_back(compute_stream, r);
    threads.emplace_back(reduce_stream, r);
  }
  for (auto& t : threads) t.join();
  if (g_failed) {
    fprintf(stderr, "a bounded wait ran out\n");
    return 2;
  }
  // every rank reduced the same staging contents: shards of one unit agree on their checksum pattern across runs
  double sum = 0.0;
  for (int r = 0; r < kWorld; ++r)
    for (int u = 0; u < kUnits; ++u)
      for (int i = 0; i < kChunk; ++i) sum += g_rank[r].grad[u][i];
  printf("checksum %.6f\n", sum);
  return 0;
}
