"""DCP checkpoint of the native model -> consolidated Hugging Face safetensors.
``python -m torchtitan_b200.scripts.checkpoint_conversion.convert_to_hf <dcp_dir> <hf_dir> --model_name llama3 --model_flavor 8B
--hf_assets_path ./assets/hf/Llama-3.1-8B --export_dtype bfloat16``. Parity: scripts/checkpoint_conversion/convert_to_hf.py."""

import argparse
import importlib
from pathlib import Path

import torch
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint import HuggingFaceStorageWriter

from torchtitan_b200.components.checkpoint import ModelWrapper
from torchtitan_b200.config import TORCH_DTYPE_MAP


@torch.inference_mode()
def convert_to_hf(input_dir, output_dir, model_name, model_flavor, hf_assets_path, export_dtype):
    spec = importlib.import_module(f"torchtitan_b200.models.{model_name}").model_registry(model_flavor)
    with torch.device("cpu"):
        model = spec.model.build()
    wrapper = ModelWrapper(model)
    adapter = spec.state_dict_adapter(spec.model, hf_assets_path)
    assert adapter is not None, "trying to convert checkpoint from DCP to HF safetensors format, but sd_adapter is not provided."
    sd = wrapper._get_state_dict()
    dcp.load(sd, checkpoint_id=str(input_dir))
    hf_sd = adapter.to_hf(sd)
    writer = HuggingFaceStorageWriter(path=str(output_dir), save_distributed=True,
                                      fqn_to_index_mapping=getattr(adapter, "fqn_to_index_mapping", None),
                                      enable_consolidation=True, thread_count_consolidation=5)
    dtype = TORCH_DTYPE_MAP[export_dtype]
    if dtype != torch.float32:
        hf_sd = {k: v.to(dtype) for k, v in hf_sd.items()}
    dcp.save(hf_sd, storage_writer=writer)


if __name__ == "__main__":
    p = argparse.ArgumentParser(description="Convert DCP weights to HF format.")
    p.add_argument("input_dir", type=Path)
    p.add_argument("output_dir", type=Path)
    p.add_argument("--hf_assets_path", type=Path, default="./assets/hf/Llama-3.1-8B")
    p.add_argument("--model_name", type=str, nargs="?", default="llama3")
    p.add_argument("--model_flavor", type=str, nargs="?", default="8B")
    p.add_argument("--export_dtype", type=str, nargs="?", choices=["float16", "bfloat16", "float32"], default="float32")
    a = p.parse_args()
    convert_to_hf(a.input_dir, a.output_dir, a.model_name, a.model_flavor, a.hf_assets_path, a.export_dtype)
