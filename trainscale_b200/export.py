"""Model export: merged safetensors in HuggingFace layout, GGUF (through an installed llama.cpp converter), a serving
config for this framework's / a vLLM-style engine, and hub upload.

After data_pipeline/trainer/export.py:72-452 (`merge_lora_weights`, `save_safetensors`, `export_to_gguf`,
`create_vllm_config`, `push_to_hub`, `export_model`).
"""
from __future__ import annotations

import json
import shutil
import subprocess
import sys
from pathlib import Path

import torch

from .core.errors import HubError
from .hub import HubManager, ModelSerializer, generate_model_card
from .utils.refargs import ANY, reference_kwargs


def merge_lora_weights(model):
    from .lora import merge_and_unload
    return merge_and_unload(model)


def _shard_gb(size) -> float:
    """"5GB" / "500MB" / a number of bytes -> GiB."""
    if isinstance(size, str):
        t = size.strip().upper()
        for unit, f in (("GB", 1.0), ("MB", 1 / 1024), ("KB", 1 / 1024 ** 2)):
            if t.endswith(unit):
                return float(t[:-2]) * f
        return float(t) / 2 ** 30
    return float(size) / 2 ** 30


@reference_kwargs(output_dir="out_dir")
def save_safetensors(model, out_dir, max_shard_gb: float = 5.0, tokenizer=None, *, max_shard_size=None) -> Path:
    """Sharded safetensors (+ index, config.json, tokenizer files) under `out_dir`.  `max_shard_size` is the
    reference's spelling of the shard limit: "5GB", "500MB" or a number of bytes."""
    if max_shard_size is not None:
        max_shard_gb = _shard_gb(max_shard_size)
    out = Path(out_dir)
    sd = model.to_hf_state_dict() if hasattr(model, "to_hf_state_dict") else model.state_dict()
    ModelSerializer(int(max_shard_gb * 2 ** 30)).save(sd, out)
    if hasattr(model, "hf_config_dict"):
        (out / "config.json").write_text(json.dumps(model.hf_config_dict(), indent=2))
    tok = getattr(tokenizer, "tokenizer", tokenizer)
    if tok is not None and hasattr(tok, "save_pretrained"):
        tok.save_pretrained(str(out))
    return out


def export_to_gguf(model_dir=None, out_file=None, quantization: str = "f16", converter: str | None = None, *, model=None,
                   tokenizer=None, output_dir=None) -> Path:
    """Needs llama.cpp's `convert_hf_to_gguf.py` (path in `converter` or on PATH); raises HubError when absent.
    The reference's form `export_to_gguf(model, tokenizer, output_dir, quantization)` (a module first) saves the model
    as safetensors under `output_dir` and converts that folder to `output_dir/model-<quantization>.gguf`."""
    if model is not None or isinstance(model_dir, torch.nn.Module):
        model = model if model is not None else model_dir
        tokenizer = tokenizer if tokenizer is not None else (out_file if not isinstance(out_file, (str, Path)) else None)
        output_dir = output_dir if output_dir is not None else (quantization if converter in
                                                                ("f16", "bf16", "q8_0", "f32", "q4_k_m", "q5_k_m") else None)
        if output_dir is None:
            raise ValueError("export_to_gguf(model, tokenizer, output_dir, quantization): output_dir is required")
        if converter in ("f16", "bf16", "q8_0", "f32", "q4_k_m", "q5_k_m"):
            quantization, converter = converter, None
        model_dir = save_safetensors(model, output_dir, tokenizer=tokenizer)
        out_file = Path(output_dir) / f"model-{quantization}.gguf"
    conv = converter or shutil.which("convert_hf_to_gguf.py") or shutil.which("convert-hf-to-gguf.py")
    if conv is None:
        raise HubError("GGUF export needs llama.cpp's convert_hf_to_gguf.py; pass converter=<path>")
    out = Path(out_file)
    out.parent.mkdir(parents=True, exist_ok=True)
    outtype = {"f16": "f16", "bf16": "bf16", "q8_0": "q8_0", "f32": "f32"}.get(quantization, "f16")
    subprocess.run([sys.executable, conv, str(model_dir), "--outfile", str(out), "--outtype", outtype], check=True)
    return out


@reference_kwargs(model_path="model_dir")
def create_vllm_config(model_dir, tensor_parallel_size: int | str = 1, max_model_len: int = 8192, dtype: str = "bfloat16",
                       gpu_memory_utilization: float = 0.9, *, output_dir=None) -> Path:
    """Writes serving_config.json (engine arguments for this framework's server or vLLM) into `output_dir`, by default
    the model folder; `create_vllm_config(model_path, output_dir)` is the reference's positional form."""
    if isinstance(tensor_parallel_size, (str, Path)):             # (model_path, output_dir)
        output_dir, tensor_parallel_size = tensor_parallel_size, 1
    cfg = {"model": str(model_dir), "tensor_parallel_size": tensor_parallel_size, "max_model_len": max_model_len,
           "dtype": dtype, "gpu_memory_utilization": gpu_memory_utilization, "enable_prefix_caching": True}
    target = Path(output_dir if output_dir is not None else model_dir)
    target.mkdir(parents=True, exist_ok=True)
    p = target / "serving_config.json"
    p.write_text(json.dumps(cfg, indent=2))
    return p


def push_to_hub(folder=None, repo_id: str | None = None, token: str | None = None, private: bool = False, *, model=None,
                tokenizer=None, commit_message: str = "export") -> str | None:
    """Upload a folder.  The reference's form `push_to_hub(model, tokenizer, repo_id, token, private, commit_message)`
    (a module first) saves the model and tokenizer to a temporary folder and uploads that."""
    if model is not None or isinstance(folder, torch.nn.Module):
        import tempfile
        if model is None:                                 # positional: (model, tokenizer, repo_id, token?)
            model, tokenizer, repo_id, token = folder, repo_id, token, (private if isinstance(private, str) else None)
            private = False if isinstance(private, str) else private
        with tempfile.TemporaryDirectory(prefix="ts_export_") as tmp:
            save_safetensors(model, tmp, tokenizer=tokenizer)
            return HubManager(repo_id, token, private).push(tmp, commit_message)
    return HubManager(repo_id, token, private).push(folder, commit_message)


def export_model(model, out_dir, fmt: str = "safetensors", tokenizer=None, merge_lora: bool = True,
                 hub_model_id: str | None = None, hub_token: str | None = None, **kw) -> Path:
    if merge_lora and any("lora_" in n for n, _ in model.named_parameters()):
        model = merge_lora_weights(model)
    out = Path(out_dir)
    if fmt in ("safetensors", "vllm", "sglang") or fmt.startswith("gguf"):
        save_safetensors(model, out, tokenizer=tokenizer)
        if fmt in ("vllm", "sglang"):
            create_vllm_config(out, **{k: v for k, v in kw.items() if k in ("tensor_parallel_size", "max_model_len")})
        if fmt.startswith("gguf"):
            export_to_gguf(out, out / f"model-{fmt.replace('gguf_', '')}.gguf", fmt.replace("gguf_", ""), kw.get("converter"))
    elif fmt == "pytorch":
        out.mkdir(parents=True, exist_ok=True)
        torch.save({k: v.detach().cpu() for k, v in model.state_dict().items()}, out / "pytorch_model.bin")
    else:
        raise ValueError(f"unknown export format {fmt!r}")
    (out / "README.md").write_text(generate_model_card(out.name, config=getattr(model, "hf_config_dict", dict)()))
    if hub_model_id:
        push_to_hub(out, hub_model_id, hub_token)
    return out


def prepare_for_vllm(model_path: str, tensor_parallel_size: int = 1, dtype: str = "auto") -> dict:
    """Keyword arguments for `vllm.LLM(...)` serving an exported directory (data_pipeline/trainer/export.py:278-296)."""
    return {"model": str(model_path), "tensor_parallel_size": int(tensor_parallel_size), "dtype": dtype,
            "trust_remote_code": True, "gpu_memory_utilization": 0.9}


def unmerge_lora_weights(model, lora_state_dict: dict):
    """Undo a merge: subtract scaling * B @ A from every module whose adapter tensors are in `lora_state_dict`
    (`<module>.lora_A.weight`, `<module>.lora_B.weight`, optional `<module>.scaling`), in place
    (data_pipeline/trainer/export.py:111-130)."""
    import torch
    with torch.no_grad():
        for name, module in model.named_modules():
            a, b = lora_state_dict.get(f"{name}.lora_A.weight"), lora_state_dict.get(f"{name}.lora_B.weight")
            w = getattr(module, "weight", None)
            if a is None or b is None or w is None:
                continue
            scale = float(lora_state_dict.get(f"{name}.scaling", 1.0))
            w.sub_((scale * (b.float() @ a.float())).to(w.dtype).to(w.device))
    return model
