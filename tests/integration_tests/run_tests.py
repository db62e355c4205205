"""Run a suite of integration cases as real training jobs.

    python -m tests.integration_tests.run_tests <output_dir> [--test_suite features] [--test_name all] [--ngpu 8]
                                                [--cpu] [--dry_run] [--keep_going] [--extra "--training.steps 2"]

Each case becomes one ``run_train.sh`` invocation per override set (``NGPU``, ``MODULE``, ``CONFIG`` in the environment,
flags on the command line), all in the case's own dump folder ``<output_dir>/<test_name>``; a non-zero exit fails the
run. ``--cpu`` leaves out the cases that need a GPU (the jobs then run on gloo ranks); ``--dry_run`` validates every
case (flags parse into the configuration, degrees fit the rank count) without launching anything.
Reference: tests/integration_tests/run_tests.py:25-150."""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
import time

from . import OverrideDefinitions

_REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def suites() -> dict:
    from . import b200, experiments, features, flux, models

    return {
        "features": features.build_features_test_list, "models": models.build_model_tests_list,
        "b200": b200.build_b200_tests_list, "flux": flux.build_flux_test_list, "vlm": experiments.build_vlm_test_list,
        "autoparallel": experiments.build_autoparallel_test_list,
        "transformers_modeling_backend": experiments.build_transformers_backend_test_list,
        "ft": experiments.build_ft_test_list, "graph_trainer": experiments.build_graph_trainer_test_list,
    }


def command(case: OverrideDefinitions, i: int, dump: str, extra: list[str]) -> tuple[dict, list[str]]:
    """Environment additions and argv of override set ``i``; ``{dump}`` in a flag expands to the case's dump folder."""
    env = {"NGPU": str(case.ngpu), "MODULE": case.module, "CONFIG": case.config, "LOG_RANK": "0"}
    if i < len(case.env):
        env.update(case.env[i])
    flags = [f.replace("{dump}", dump) for f in case.flags(i)]
    return env, [os.path.join(_REPO, "run_train.sh"), "--dump_folder", dump, *flags, *_without(extra, flags)]


def _without(extra: list[str], flags: list[str]) -> list[str]:
    """``extra`` minus the options the case sets itself (the case wins): an option is a ``--name`` and the values after it."""
    mine = {f.split("=")[0] for f in flags if f.startswith("--")}
    out, keep = [], True
    for tok in extra:
        if tok.startswith("--"):
            keep = tok.split("=")[0] not in mine
        if keep:
            out.append(tok)
    return out


def validate(case: OverrideDefinitions, extra: list[str] = ()) -> None:
    """Parse every override set into the case's configuration and check that the parallel degrees fit ``ngpu``."""
    from torchtitan_b200.config.manager import ConfigManager

    for i in range(len(case.override_args)):
        flags = [f.replace("{dump}", "/tmp/x") for f in case.flags(i)]
        cfg = ConfigManager().parse_args(["--module", case.module, "--config", case.config, *flags, *extra])
        if case.module == "autoparallel":        # the planner picks the degrees at start-up
            continue
        p = cfg.parallelism
        fixed = (p.data_parallel_replicate_degree * p.context_parallel_degree * p.tensor_parallel_degree
                 * p.pipeline_parallel_degree)
        shard = p.data_parallel_shard_degree
        if shard == -1:
            assert case.ngpu % fixed == 0, f"{case.test_name}: {case.ngpu} ranks do not divide by the fixed degrees ({fixed})"
        else:
            assert fixed * shard == case.ngpu, f"{case.test_name}: degrees give {fixed * shard} ranks, case asks for {case.ngpu}"


def run_case(case: OverrideDefinitions, output_dir: str, extra: list[str], timeout: float | None = None) -> float:
    dump = os.path.join(output_dir, case.test_name)
    t0 = time.perf_counter()
    for i in range(len(case.override_args)):
        add, argv = command(case, i, dump, extra)
        print(f"===== {case.test_name} [{i + 1}/{len(case.override_args)}] ({case.test_descr}): "
              f"NGPU={case.ngpu} MODULE={case.module} CONFIG={case.config} {' '.join(argv[1:])}", flush=True)
        res = subprocess.run(argv, env={**os.environ, **add}, cwd=_REPO, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                             text=True, timeout=timeout)
        if res.returncode != 0:
            print(res.stdout[-6000:])
            raise RuntimeError(f"integration case {case.test_name!r} failed (exit code {res.returncode}) on override set {i}")
    return time.perf_counter() - t0


def select(suite: str, test_name: str, ngpu: int, cpu: bool) -> tuple[list[OverrideDefinitions], list[tuple[str, str]]]:
    table = suites()
    if suite not in table:
        raise SystemExit(f"unknown --test_suite {suite!r}; available: {sorted(table)}")
    cases, skipped = [], []
    for c in table[suite]():
        if test_name != "all" and c.test_name != test_name:
            continue
        why = ("disabled" if c.disabled else "needs a GPU" if (cpu and c.needs_gpu)
               else f"needs {c.ngpu} ranks, {ngpu} given" if c.ngpu > ngpu else None)
        (skipped.append((c.test_name, why)) if why else cases.append(c))
    if test_name != "all" and not cases and not skipped:
        raise SystemExit(f"no case named {test_name!r} in suite {suite!r}")
    return cases, skipped


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("output_dir")
    ap.add_argument("--test_suite", default="features")
    ap.add_argument("--test_name", default="all")
    ap.add_argument("--ngpu", type=int, default=8)
    ap.add_argument("--cpu", action="store_true", help="leave out the cases that need a GPU")
    ap.add_argument("--dry_run", action="store_true", help="validate the cases, launch nothing")
    ap.add_argument("--keep_going", action="store_true", help="run the remaining cases after a failure; exit 1 at the end")
    ap.add_argument("--extra", default="", help="flags appended to every job, as one string")
    a = ap.parse_args(argv)
    extra = a.extra.split()
    cases, skipped = select(a.test_suite, a.test_name, a.ngpu, a.cpu)
    for name, why in skipped:
        print(f"skipped {name}: {why}")
    os.makedirs(a.output_dir, exist_ok=True)
    lighthouse = None
    if a.test_suite == "ft" and cases and not a.dry_run and not os.environ.get("TT_LIGHTHOUSE"):
        # fault-tolerant jobs register with a quorum service: run one for the duration of the suite
        from torchtitan_b200.experiments.ft.lighthouse import Lighthouse

        lighthouse = Lighthouse()
        os.environ["TT_LIGHTHOUSE"] = lighthouse.address
    failed = []
    for c in cases:
        validate(c, extra)
        if a.dry_run:
            print(f"valid   {c.test_name}: {c.test_descr}")
            continue
        try:
            dt = run_case(c, a.output_dir, extra)
            print(f"passed  {c.test_name} in {dt:.0f} s", flush=True)
        except RuntimeError as e:
            if not a.keep_going:
                raise
            print(f"FAILED  {c.test_name}: {e}", flush=True)
            failed.append(c.test_name)
    if lighthouse is not None:
        lighthouse.shutdown()
        os.environ.pop("TT_LIGHTHOUSE", None)
    if failed:
        print(f"{len(failed)} failed: {failed}")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
