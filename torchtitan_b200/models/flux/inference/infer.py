"""Generate images for a file of prompts with a trained FLUX checkpoint.

``torchrun ... -m torchtitan_b200.models.flux.inference.infer --module flux --config flux_debugmodel --checkpoint.enable
--checkpoint.exclude_from_loading=lr_scheduler,dataloader,optimizer --inference.prompts_path prompts.txt``

The trainer object is reused for its model, frozen encoders, autoencoder and checkpoint loading; prompts are dealt
round-robin to the ranks, each rank samples its share in batches of ``--inference.local_batch_size`` at
``--inference.img_size`` with the ``--validation.*`` sampling options and writes
``<dump_folder>/<inference.save_img_folder>/image_prompt<i>_rank<r>.png``. Under FSDP every rank must run the same
number of forward passes, so a rank with fewer prompts than the others repeats its last batch without saving it
(the reference refuses fewer prompts than ranks and otherwise leaves the counts uneven,
torchtitan/models/flux/inference/infer.py:19-92).
"""

from __future__ import annotations

import os

import torch

from torchtitan_b200.config import ConfigManager
from torchtitan_b200.tools.logging import init_logger, logger

from ..tokenizer import build_flux_tokenizer
from ..trainer import FluxTrainer
from .sampling import generate_image, save_image

__all__ = ["inference", "read_prompts", "share_of"]


def read_prompts(path: str) -> list[str]:
    with open(path) as f:
        return [line.strip() for line in f if line.strip()]


def share_of(n_prompts: int, rank: int, world: int, batch: int) -> tuple[list[int], int]:
    """(global indices of this rank's prompts, number of batches every rank runs)."""
    mine = list(range(rank, n_prompts, world))
    most = -(-n_prompts // world)
    return mine, -(-most // batch)


@torch.no_grad()
def inference(config: FluxTrainer.Config) -> list[str]:
    trainer = FluxTrainer(config)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    prompts = read_prompts(config.inference.prompts_path)
    if len(prompts) < world:
        raise ValueError(f"Number of prompts ({len(prompts)}) must be >= number of ranks ({world}). "
                         "FSDP all-gather will hang if some ranks have no prompts to process.")
    trainer.checkpointer.load(step=config.checkpoint.load_step)
    e, dl = config.encoder, config.dataloader
    t5_tok, clip_tok = build_flux_tokenizer(
        t5_path=getattr(dl, "t5_tokenizer_path", None) or e.t5_encoder, clip_path=getattr(dl, "clip_tokenizer_path", None) or e.clip_encoder,
        t5_max_length=getattr(dl, "t5_max_length", e.max_t5_encoding_len), clip_max_length=getattr(dl, "clip_max_length", 77),
        test_mode=e.test_mode or getattr(dl, "test_tokenizer", False) or e.random_init)
    model = trainer.model_parts[0]
    model.eval()
    bs = config.inference.local_batch_size
    size = 16 * (config.inference.img_size // 16)
    out_dir = os.path.join(config.dump_folder, config.inference.save_img_folder)
    mine, n_batches = share_of(len(prompts), rank, world, bs)
    if rank == 0:
        logger.info(f"Starting inference: {len(prompts)} prompts on {world} rank(s), {n_batches} batch(es) of {bs} each")
    written = []
    for b in range(n_batches):
        ids = mine[b * bs : (b + 1) * bs]
        filler = not ids                                   # keep the collectives of sharded models in step
        if filler:
            ids = mine[-bs:]
        with trainer.maybe_enable_amp:
            images = generate_image(trainer.device, trainer._dtype, model=model, autoencoder=trainer.autoencoder,
                                    clip_encoder=trainer.clip_encoder, t5_encoder=trainer.t5_encoder,
                                    prompt=[prompts[i] for i in ids], clip_tokenizer=clip_tok, t5_tokenizer=t5_tok,
                                    job_config=config, height=size, width=size, seed=None)
        if filler:
            continue
        for img, i in zip(images, ids):
            written.append(save_image(img, out_dir, f"image_prompt{i}_rank{rank}.png", prompt=prompts[i]))
    trainer.close()
    return written


if __name__ == "__main__":
    init_logger()
    cfg = ConfigManager().parse_args()
    try:
        inference(cfg)
    finally:
        if torch.distributed.is_initialized():
            torch.distributed.destroy_process_group()
