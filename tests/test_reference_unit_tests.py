"""The reference's own unit tests, run against this package.

With ``$TORCHTITAN_REFERENCE`` pointing at a checkout of the reference (one that has ``tests/unit_tests``), its unit-test
files are collected in a child pytest process in which ``import torchtitan`` resolves to ``torchtitan_b200``
(``reference_alias_plugin.py``). They cover the public surface a user of the reference relies on: configuration manager
and registries, checkpoint manager, dataloaders and their resumption, the FLUX dataset registry, losses, LR schedules,
model converters, module protocol, RoPE / RMSNorm / linear / embedding layers, activation checkpointing, seeds,
permutation indices, model specs. Left out, with the reason:

* cases that assert the reference's private structure rather than behaviour (``_EXCLUDED``);
* ``test_compile_moe.py``: the ``torch.compile`` wrapper of MoE layers; this framework has no compiler path;
* ``test_download_hf_assets.py`` / ``test_tokenizer.py``: import the checkout's top-level ``scripts`` package and
  download from the Hugging Face hub.

Skipped when no checkout is given (the offline install under ``baseline/_ref`` carries the package but not its tests).
"""

import os
import subprocess
import sys

import pytest

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.environ.get("TORCHTITAN_REFERENCE", "")
_UT = os.path.join(_REF, "tests", "unit_tests")

pytestmark = pytest.mark.skipif(not os.path.isdir(_UT), reason="no reference checkout with tests/unit_tests in $TORCHTITAN_REFERENCE")

_IGNORED_FILES = ["test_compile_moe.py", "test_download_hf_assets.py", "test_tokenizer.py"]
_EXCLUDED = {
    # patches a class attribute of the reference's checkpoint module that this implementation does not have
    "test_checkpoint.py::TestCheckpointManager::test_async_save_with_pinned_mem_sets_staging_flag": "DefaultStager",
    # calls a private helper of the reference's ConfigManager
    "test_config_manager.py::TestConfigManager::test_extend_trainer_config_directly": "_merge_configs",
    # read the private dict of eagerly built meshes; here meshes and groups are built on first use
    "test_parallel_dims.py::TestParallelDimsMeshOperations::test_get_mesh_lazy_initialization": "_meshes",
    "test_parallel_dims.py::TestParallelDimsMeshOperations::test_single_rank_mesh_operations": "_meshes",
    "test_parallel_dims.py::TestParallelDimsWorld8MeshOperations::test_world_size_8_mesh_operations": "_meshes",
    # builds ParallelDims with an expert degree that does not divide the ranks; rejected at construction here
    "test_parallel_dims.py::TestParallelDimsMeshOperations::test_expert_parallelism_validation": "ep=3 on 4 ranks",
}


def test_reference_unit_tests_pass_against_this_package(tmp_path):
    # the tests open ``tests/assets/...`` relative to the working directory
    assets = tmp_path / "tests" / "assets"
    assets.mkdir(parents=True)
    for src in (os.path.join(_REF, "tests", "assets"), os.path.join(_HERE, "assets")):
        for name in sorted(os.listdir(src)) if os.path.isdir(src) else ():
            if not (assets / name).exists():
                os.symlink(os.path.join(src, name), assets / name)
    # a copy keeps byte-code and cache files out of the checkout
    ut = tmp_path / "ut"
    ut.mkdir()
    for name in sorted(os.listdir(_UT)):
        if name.endswith(".py") and name not in _IGNORED_FILES:
            (ut / name).write_bytes(open(os.path.join(_UT, name), "rb").read())
    argv = [sys.executable, "-m", "pytest", "ut", "-q", "--no-header", "-p", "no:cacheprovider", "-p", "reference_alias_plugin",
            "--rootdir", str(tmp_path)]
    for case in _EXCLUDED:
        argv += ["--deselect", "ut/" + case]
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([_HERE, os.path.dirname(_HERE), env.get("PYTHONPATH", "")])
    env.pop("TORCHTITAN_REFERENCE", None)
    res = subprocess.run(argv, cwd=tmp_path, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1800)
    tail = res.stdout[-4000:]
    assert res.returncode == 0, tail
    assert " passed" in tail and " failed" not in tail and " error" not in tail.lower().split("warnings summary")[-1], tail
