"""Hugging Face safetensors folder -> DCP checkpoint of the native model.
``python -m torchtitan_b200.scripts.checkpoint_conversion.convert_from_hf <hf_dir> <dcp_dir> --model_name llama3 --model_flavor 8B``
Parity: scripts/checkpoint_conversion/convert_from_hf.py."""

import argparse
import importlib
from pathlib import Path

import torch
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint import HuggingFaceStorageReader

from torchtitan_b200.components.checkpoint import ModelWrapper


@torch.inference_mode()
def convert_from_hf(input_dir, output_dir, model_name, model_flavor):
    spec = importlib.import_module(f"torchtitan_b200.models.{model_name}").model_registry(model_flavor)
    with torch.device("cpu"):
        model = spec.model.build()
    wrapper = ModelWrapper(model)
    adapter = spec.state_dict_adapter(spec.model, None)
    assert adapter is not None, "trying to convert checkpoint from HF to DCP safetensors format, but sd_adapter is not provided."
    hf_sd = adapter.to_hf(wrapper._get_state_dict())          # empty tensors with the Hugging Face names/shapes
    dcp.load(hf_sd, storage_reader=HuggingFaceStorageReader(path=str(input_dir)))
    dcp.save(adapter.from_hf(hf_sd), checkpoint_id=str(output_dir))


if __name__ == "__main__":
    p = argparse.ArgumentParser(description="Convert HF checkpoint to DCP format.")
    p.add_argument("input_dir", type=Path)
    p.add_argument("output_dir", type=Path)
    p.add_argument("--model_name", type=str, nargs="?", default="llama3")
    p.add_argument("--model_flavor", type=str, nargs="?", default="8B")
    a = p.parse_args()
    convert_from_hf(a.input_dir, a.output_dir, a.model_name, a.model_flavor)
