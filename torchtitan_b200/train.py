"""Entry point: ``python -m torchtitan_b200.train --module llama3 --config llama3_8b [--a.b v]``.

Parity: torchtitan/train.py:16-64 (parse config, build the trainer, optionally write a seed
checkpoint at step 0 and stop, otherwise train; always tear the process group down)."""

import os

import torch

from torchtitan_b200.config.manager import ConfigManager
from torchtitan_b200.tools.logging import init_logger, logger


def main() -> None:
    init_logger()
    import torchtitan_b200

    logger.info(f"torchtitan_b200 version: {torchtitan_b200.__version__}")
    config = ConfigManager().parse_args()
    trainer = None
    try:
        trainer = config.build()
        if config.checkpoint.create_seed_checkpoint:
            assert int(os.environ.get("WORLD_SIZE", "1")) == 1, "Must create seed checkpoint using a single device, to disable sharding."
            assert config.checkpoint.enable, "Must enable checkpointing when creating a seed checkpoint."
            trainer.checkpointer.save(curr_step=0, last_step=True)
            logger.info("Created seed checkpoint")
        elif config.comm.mode == "fake_backend":
            logger.info("fake_backend dry run: configuration, meshes and parallelisation validated")
        else:
            trainer.train()
    except Exception:
        if trainer is not None:
            trainer.close()
        raise
    else:
        trainer.close()
        if torch.distributed.is_initialized():
            torch.distributed.destroy_process_group()
        logger.info("Process group destroyed")


if __name__ == "__main__":
    main()
