"""Periodic validation: on step 1 and every ``freq`` steps the model scores ``steps`` batches of the validation
loader and the mean token loss goes to the metrics processor.

Same contract as torchtitan/components/validate.py:30-314 (per batch ``loss_sum / global_valid_tokens``, averaged over
the batches, summed over the ``loss`` mesh; training context, AMP, context-parallel sharding and the pipeline's ``eval``
are reused). The pass itself is organised differently: batches come from a bounded generator, each is scored by one of
two scorers (pipeline / single model part), and the running mean stays on the device, so a validation pass reads one
number back instead of synchronising once per batch."""

from __future__ import annotations

import contextlib
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

    # ------------------------------------------------------------------ one pass
    def _batches(self):
        """At most ``steps`` batches (all of them for -1), already on the device."""
        dev = utils.device_type
        for n, (input_dict, labels) in enumerate(self.validation_dataloader):
            if self.config.steps != -1 and n >= self.config.steps:
                return
            self.metrics_processor.ntokens_since_last_log += labels.numel()
            yield {k: v.to(dev) for k, v in input_dict.items()}, labels.to(dev)

    def _score_pipeline(self, inputs, labels, extra_inputs, extra_kwargs) -> torch.Tensor:
        last = self.pp_has_last_stage
        targets, losses = (labels, []) if last else (None, None)
        first_args = (inputs,) if self.pp_has_first_stage else ()
        first_kwargs = extra_inputs if self.pp_has_first_stage else {}
        with self.validation_context():
            self.pp_schedule.eval(*first_args, **first_kwargs, **extra_kwargs, target=targets, losses=losses)
        if not last:          # ranks without the last stage contribute nothing; the loss mesh sums the real value in
            return torch.zeros((), device=utils.device_type) - 1.0
        return torch.stack(losses).sum().to(utils.device_type)

    def _score_single(self, model, inputs, labels, extra_inputs, extra_kwargs) -> torch.Tensor:
        with self.validation_context(), self.maybe_enable_amp:
            return self.loss_fn(model(inputs, **extra_inputs, **extra_kwargs), labels)

    @contextlib.contextmanager
    def _eval_mode(self, model_parts):
        for m in model_parts:
            m.eval()
        try:
            yield
        finally:
            for m in model_parts:
                m.train()

    @torch.no_grad()
    def validate(self, model_parts: list[nn.Module], step: int) -> None:
        pd = self.parallel_dims
        batch_group = pd.get_mesh("batch").get_group() if pd.dp_enabled else None
        mean_sum, n = None, 0
        with self._eval_mode(model_parts):
            for input_dict, labels in self._batches():
                inputs, labels, extra_inputs, extra_kwargs = self.post_dataloading_process(input_dict, labels, model_parts)
                valid = (labels != IGNORE_INDEX).sum().to(torch.float32)
                if batch_group is not None:
                    torch.distributed.all_reduce(valid, group=batch_group)
                if pd.pp_enabled:
                    loss_sum = self._score_pipeline(inputs, labels, extra_inputs, extra_kwargs)
                else:
                    assert len(model_parts) == 1
                    loss_sum = self._score_single(model_parts[0], inputs, labels, extra_inputs, extra_kwargs)
                term = (loss_sum.detach() / valid).reshape(())
                mean_sum = term if mean_sum is None else mean_sum + term
                n += 1
        loss = (mean_sum if mean_sum is not None else torch.zeros((), device=utils.device_type)) / max(n, 1)
        global_avg = dist_utils.dist_sum(loss, pd.get_optional_mesh("loss")) if pd.dp_cp_enabled else loss.item()
        self.metrics_processor.log_validation(loss=global_avg, step=step)
