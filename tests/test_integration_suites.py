"""The integration suites themselves: every case must parse into its configuration and fit its rank count, names are
unique, and one save-and-resume case really runs as ``run_train.sh`` jobs on CPU ranks.

Reference: tests/integration_tests/run_tests.py (the runner) and the per-suite lists next to it."""

import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tests.integration_tests import OverrideDefinitions, run_tests  # noqa: E402


@pytest.mark.parametrize("suite", sorted(run_tests.suites()))
def test_every_case_of_the_suite_is_valid(suite):
    cases = run_tests.suites()[suite]()
    assert cases and len({c.test_name for c in cases}) == len(cases)
    for c in cases:
        assert 1 <= c.ngpu <= 8 and c.test_descr
        run_tests.validate(c)


def test_selection_and_command_line():
    cases, skipped = run_tests.select("features", "all", ngpu=2, cpu=True)
    names = {c.test_name for c in cases}
    assert "pp_1f1b" in names and "default" not in names            # the default case wants 4 ranks
    assert ("float8", "needs a GPU") in skipped and ("default", "needs 4 ranks, 2 given") in skipped
    case = OverrideDefinitions([["--checkpoint.enable", "--checkpoint.initial_load_path {dump}/hf/step-10"]], "d", "n", ngpu=2)
    env, argv = run_tests.command(case, 0, "/out/n", ["--training.steps", "2"])
    assert env["NGPU"] == "2" and env["MODULE"] == "llama3" and argv[0].endswith("run_train.sh")
    assert argv[1:] == ["--dump_folder", "/out/n", "--checkpoint.enable", "--checkpoint.initial_load_path", "/out/n/hf/step-10",
                        "--training.steps", "2"]
    # an option the case sets itself is not overridden by the extras
    _, argv = run_tests.command(OverrideDefinitions([["--training.steps 20"]], "d", "n"), 0, "/o", ["--training.steps", "2", "--x", "1"])
    assert argv[3:] == ["--training.steps", "20", "--x", "1"]
    with pytest.raises(SystemExit):
        run_tests.select("no_such_suite", "all", 8, False)
    with pytest.raises(AssertionError):
        run_tests.validate(OverrideDefinitions([["--parallelism.tensor_parallel_degree 4"]], "bad", "bad", ngpu=2))


def test_one_case_runs_end_to_end_on_cpu_ranks(tmp_path):
    rc = run_tests.main([str(tmp_path), "--test_suite", "features", "--test_name", "fsdp_reshard_always", "--ngpu", "2", "--cpu",
                         "--extra", "--training.steps 3 --training.local_batch_size 2 --training.seq_len 64"])
    assert rc == 0
