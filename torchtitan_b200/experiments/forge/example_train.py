"""A training loop written against :class:`ForgeEngine` (the engine builds, the caller steps).
``python -m torchtitan_b200.experiments.forge.example_train --module llama3 --config llama3_debugmodel`` reuses any
trainer configuration; only the sections the engine knows are taken from it.
Parity: torchtitan/experiments/forge/example_train.py:35-469."""

from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist

from torchtitan_b200.components.loss import IGNORE_INDEX
from torchtitan_b200.parallel import utils as dist_utils
from torchtitan_b200.tools.logging import init_logger, logger

from .engine import ForgeEngine


class ExampleTrainer(ForgeEngine):
    def __init__(self, config: ForgeEngine.Config, dataloader_config=None, tokenizer=None):
        super().__init__(config)
        self.tokenizer = tokenizer
        self.dataloader = None
        if dataloader_config is not None:
            self.dataloader = dataloader_config.build(
                dp_world_size=self.dp_degree, dp_rank=self.dp_rank, tokenizer=tokenizer, seq_len=config.training.seq_len,
                local_batch_size=config.training.local_batch_size, model_vocab_size=getattr(self.model_config, "vocab_size", None),
            )

    def train_step(self, batches) -> torch.Tensor:
        self.optimizers.zero_grad()
        pd = self.parallel_dims
        ntok = torch.tensor(float(sum(int((lab != IGNORE_INDEX).sum()) for _, lab in batches)), device=self.device)
        if pd.dp_enabled:
            dist.all_reduce(ntok, group=pd.get_mesh("batch").get_group())
        total = torch.zeros((), device=self.device)
        for inputs, labels in batches:
            inputs = {k: v.to(self.device) for k, v in inputs.items()}
            labels = labels.to(self.device)
            with self.train_context(), self.maybe_enable_amp:
                pred = self.model_parts[0](inputs["input"])
                loss = self.loss_fn(pred, labels) / ntok
            loss.backward()
            total += loss.detach()
        dist_utils.clip_grad_norm_([p for m in self.model_parts for p in m.parameters()], self.config.training.max_norm,
                                   foreach=True, pp_mesh=pd.get_optional_mesh("pp"), ep_enabled=pd.ep_enabled)
        self.optimizers.step()
        self.lr_schedulers.step()
        self.step += 1
        return total

    def train(self) -> list[float]:
        assert self.dataloader is not None
        it = iter(self.dataloader)
        self.checkpointer.load(step=self.config.checkpoint.load_step)
        losses = []
        while self.step < self.config.training.steps:
            self.gc_handler.run(self.step)
            batches = [next(it) for _ in range(self.gradient_accumulation_steps)]
            loss = self.train_step(batches)
            losses.append(float(loss))
            logger.info(f"step: {self.step:2}  loss: {losses[-1]:7.4f}")
            self.checkpointer.save(self.step, last_step=(self.step == self.config.training.steps))
        return losses


def engine_config_from_trainer_config(tc) -> ForgeEngine.Config:
    names = {f.name for f in dataclasses.fields(ForgeEngine.Config)}
    return ForgeEngine.Config(**{n: getattr(tc, n) for n in names if hasattr(tc, n)})


def main() -> None:
    from torchtitan_b200.config.manager import ConfigManager

    init_logger()
    tc = ConfigManager().parse_args()
    tok = tc.tokenizer.build(tokenizer_path=tc.hf_assets_path) if tc.tokenizer is not None else None
    trainer = ExampleTrainer(engine_config_from_trainer_config(tc), dataloader_config=tc.dataloader, tokenizer=tok)
    try:
        trainer.train()
    finally:
        trainer.close()
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
