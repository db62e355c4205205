"""Periodic validation. Parity: torchtitan/components/validate.py:30-314 -- runs on step 1 and
every ``freq`` steps, re-uses the training context / AMP / context-parallel sharding / pipeline
``eval``, and reports ``sum_over_steps(loss_sum / global_valid_tokens) / steps`` reduced over the
``loss`` mesh."""

from __future__ import annotations

from dataclasses import dataclass, field, replace

import torch
import torch.nn as nn

from torchtitan_b200.components.dataloader import BaseDataLoader
from torchtitan_b200.components.loss import IGNORE_INDEX
from torchtitan_b200.config.configurable import Configurable
from torchtitan_b200.hf_datasets.text_datasets import HuggingFaceTextDataLoader
from torchtitan_b200.parallel import utils as dist_utils
from torchtitan_b200.tools import utils
from torchtitan_b200.tools.logging import logger


class BaseValidator(Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        freq: int = 10

    def __init__(self, config: Config, **kwargs):
        self.config = config

    def validate(self, model_parts: list[nn.Module], step: int) -> None:
        raise NotImplementedError("validate method not implemented")

    def should_validate(self, step: int) -> bool:
        return step == 1 or step % self.config.freq == 0


class Validator(BaseValidator):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseValidator.Config):
        enable: bool = False
        steps: int = -1
        """Validation batches per run; -1 = the whole dataset (ranks may then disagree on length)."""
        dataloader: BaseDataLoader.Config = field(
            default_factory=lambda: HuggingFaceTextDataLoader.Config(dataset="c4_validation", infinite=False)
        )

        def __post_init__(self):
            assert self.steps > 0 or self.steps == -1, "validation steps must be positive or -1"

    def __init__(self, config: Config, *, parallelism, dp_world_size: int, dp_rank: int, tokenizer, parallel_dims,
                 loss_fn, validation_context, maybe_enable_amp, metrics_processor, seq_len: int,
                 local_batch_size: int, pp_schedule=None, pp_has_first_stage=None, pp_has_last_stage=None,
                 model_vocab_size=None, **kwargs):
        super().__init__(config=config)
        self.parallelism, self.tokenizer, self.parallel_dims, self.loss_fn = parallelism, tokenizer, parallel_dims, loss_fn
        dl = config.dataloader
        if hasattr(dl, "infinite"):
            dl = replace(dl, infinite=config.steps != -1)
        self.validation_dataloader = dl.build(
            dp_world_size=dp_world_size, dp_rank=dp_rank, tokenizer=tokenizer, seq_len=seq_len,
            local_batch_size=local_batch_size, model_vocab_size=model_vocab_size,
        )
        self.validation_context = validation_context
        self.maybe_enable_amp = maybe_enable_amp
        self.metrics_processor = metrics_processor
        self.pp_schedule = pp_schedule
        self.pp_has_first_stage, self.pp_has_last_stage = pp_has_first_stage, pp_has_last_stage
        if config.steps == -1:
            logger.warning(
                "Setting validation steps to -1 might cause hangs because of unequal sample counts across ranks "
                "when dataset is exhausted."
            )

    def post_dataloading_process(self, input_dict, labels, model_parts):
        from torchtitan_b200.trainer import prepare_batch

        return prepare_batch(input_dict, labels, model_parts, self.tokenizer, self.parallel_dims, self.parallelism)

    @torch.no_grad()
    def validate(self, model_parts: list[nn.Module], step: int) -> None:
        for m in model_parts:
            m.eval()
        pd = self.parallel_dims
        dev = utils.device_type
        losses_acc, n = [], 0
        for input_dict, labels in self.validation_dataloader:
            if self.config.steps != -1 and n >= self.config.steps:
                break
            self.metrics_processor.ntokens_since_last_log += labels.numel()
            input_dict = {k: v.to(dev) for k, v in input_dict.items()}
            labels = labels.to(dev)
            inputs, labels, extra_inputs, extra_kwargs = self.post_dataloading_process(input_dict, labels, model_parts)
            valid = (labels != IGNORE_INDEX).sum().to(torch.float32)
            if pd.dp_enabled:
                torch.distributed.all_reduce(valid, group=pd.get_mesh("batch").get_group())
            if pd.pp_enabled:
                with self.validation_context():
                    targets, losses = (labels, []) if self.pp_has_last_stage else (None, None)
                    if self.pp_has_first_stage:
                        self.pp_schedule.eval(inputs, **extra_inputs, **extra_kwargs, target=targets, losses=losses)
                    else:
                        self.pp_schedule.eval(**extra_kwargs, target=targets, losses=losses)
                loss_sum = torch.sum(torch.stack(losses)).to(dev) if self.pp_has_last_stage else torch.tensor([-1.0], device=dev)
            else:
                with self.validation_context():
                    assert len(model_parts) == 1
                    with self.maybe_enable_amp:
                        pred = model_parts[0](inputs, **extra_inputs, **extra_kwargs)
                        loss_sum = self.loss_fn(pred, labels)
            losses_acc.append(loss_sum.detach() / valid)
            n += 1
        loss = torch.sum(torch.stack(losses_acc)) / max(n, 1)
        if pd.dp_cp_enabled:
            global_avg = dist_utils.dist_sum(loss, pd.get_optional_mesh("loss"))
        else:
            global_avg = loss.item()
        self.metrics_processor.log_validation(loss=global_avg, step=step)
        for m in model_parts:
            m.train()
