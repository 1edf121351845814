"""Safetensors reader + ModelOpt NVFP4 checkpoint rules behind the command line's --hf-model-dir / --nvfp4-tensor /
--validate-nvfp4-model flags (host C++: qwen35x_b200/csrc/host/nvfp4_checkpoint.cpp), on checkpoints written here
in the layout the reference expects (src/weights/modelopt_nvfp4.cpp:30-145): per quantised linear layer a U8 weight
[N, K/2], an F8_E4M3 weight_scale [N, K/16] and scalar F32 weight_scale_2 / input_scale."""
import json
import re
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest

from helpers import make_weight

CLI = Path(__file__).resolve().parent.parent / "qwen35x_b200" / "_lib" / "q35b"
QUANT_CONFIG = {"producer": {"name": "modelopt"},
                "quantization": {"quant_algo": "NVFP4", "kv_cache_quant_algo": None, "group_size": 16, "exclude_modules": ["lm_head"]}}


def run(*args):
    return subprocess.run([str(CLI), *map(str, args)], capture_output=True, text=True, timeout=300)


def write_safetensors(path: Path, tensors: dict, metadata=None) -> None:
    """tensors: name -> (dtype string, shape, bytes)."""
    header, blobs, off = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, (dtype, shape, data) in tensors.items():
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + len(data)]}
        blobs.append(data)
        off += len(data)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * ((8 - len(text) % 8) % 8)
    path.write_bytes(struct.pack("<Q", len(text)) + text + b"".join(blobs))


def family(base: str, n: int, k: int, seed: int, input_scale: float = 1.0):
    _, codes, scales, s2 = make_weight(n, k, seed=seed)
    return {base + ".weight": ("U8", (n, k // 2), codes.tobytes()),
            base + ".weight_scale": ("F8_E4M3", (n, k // 16), scales.tobytes()),
            base + ".weight_scale_2": ("F32", (), struct.pack("<f", s2)),
            base + ".input_scale": ("F32", (), struct.pack("<f", input_scale))}, (codes, scales, s2)


def module_bases(layers: int, interval: int):
    out = []
    for i in range(layers):
        b = f"model.language_model.layers.{i}."
        out += [b + "mlp.gate_proj", b + "mlp.up_proj", b + "mlp.down_proj"]
        if (i + 1) % interval == 0:
            out += [b + "self_attn." + p for p in ("q_proj", "k_proj", "v_proj", "o_proj")]
        else:
            out += [b + "linear_attn." + p for p in ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a", "out_proj")]
    return out


def make_checkpoint(root: Path, layers=2, interval=2, sharded=True, mutate=None):
    root.mkdir(parents=True, exist_ok=True)
    tensors = {}
    for j, base in enumerate(module_bases(layers, interval)):
        fam, _ = family(base, 32, 64, seed=j)
        tensors.update(fam)
    tensors["model.language_model.embed_tokens.weight"] = ("BF16", (8, 4), bytes(64))
    if mutate:
        mutate(tensors)
    if sharded:
        names = list(tensors)
        half = len(names) // 2
        shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
        weight_map = {}
        for fname, ns in shards.items():
            write_safetensors(root / fname, {n: tensors[n] for n in ns}, metadata={"format": "pt"})
            weight_map.update({n: fname for n in ns})
        (root / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": 1}, "weight_map": weight_map}))
    else:
        write_safetensors(root / "model.safetensors", tensors, metadata={"format": "pt", "note": 'a "quoted" {brace}'})
    (root / "hf_quant_config.json").write_text(json.dumps(QUANT_CONFIG, indent=2))
    return root


@pytest.mark.parametrize("sharded", [True, False])
def test_validation_passes(engine, tmp_path, sharded):
    root = make_checkpoint(tmp_path / "ckpt", sharded=sharded)
    for extra in ([], ["--expect-layers", 2, "--full-attention-interval", 2]):
        r = run("--validate-nvfp4-model", "--hf-model-dir", root, *extra)
        assert r.returncode == 0, r.stderr
        assert "ModelOpt NVFP4 validation passed" in r.stdout
        assert re.search(r"quantized_modules: 15\b", r.stdout) and re.search(r"group_size: 16\b", r.stdout)
        assert re.search(r"fp8_scale_tensors: 15\b", r.stdout)


def test_validation_failures(engine, tmp_path):
    def expect(root, text, *extra):
        r = run("--validate-nvfp4-model", "--hf-model-dir", root, *extra)
        assert r.returncode == 10 and text in r.stderr, (r.stdout, r.stderr)

    base = "model.language_model.layers.0.mlp.down_proj"
    expect(tmp_path / "missing", "Could not open file")

    def wrong_dtype(t):
        d, s, b = t[base + ".weight"]
        t[base + ".weight"] = ("I8", s, b)
    expect(make_checkpoint(tmp_path / "a", mutate=wrong_dtype), f"Tensor '{base}.weight' has dtype I8 (expected U8).")

    def wrong_scale_shape(t):
        d, s, b = t[base + ".weight_scale"]
        t[base + ".weight_scale"] = (d, (s[0] * 2, s[1] // 2), b)
    expect(make_checkpoint(tmp_path / "b", mutate=wrong_scale_shape), "does not match expected [32,4].")

    def vector_input_scale(t):
        t[base + ".input_scale"] = ("F32", (1,), struct.pack("<f", 1.0))
    expect(make_checkpoint(tmp_path / "c", mutate=vector_input_scale), f"Tensor '{base}.input_scale' must be scalar F32.")

    def drop_scale2(t):
        del t[base + ".weight_scale_2"]
    expect(make_checkpoint(tmp_path / "d", mutate=drop_scale2), f"Tensor '{base}.weight_scale_2' not found in model.safetensors.index.json")
    # a layer the model should have is missing entirely
    expect(make_checkpoint(tmp_path / "e", layers=1), "layers.1.mlp.gate_proj.weight' not found", "--expect-layers", 2,
           "--full-attention-interval", 2)
    for key, value, text in (("quant_algo", "FP8", "does not declare quant_algo=NVFP4"), ("group_size", 32, "does not declare group_size=16"),
                             ("kv_cache_quant_algo", "FP8", "must leave kv_cache_quant_algo null")):
        root = make_checkpoint(tmp_path / ("q_" + key))
        cfg = json.loads(json.dumps(QUANT_CONFIG))
        cfg["quantization"][key] = value
        (root / "hf_quant_config.json").write_text(json.dumps(cfg))
        expect(root, text)
    # a truncated header is an error, not a crash
    root = make_checkpoint(tmp_path / "t", sharded=False)
    blob = (root / "model.safetensors").read_bytes()
    (root / "model.safetensors").write_bytes(blob[:40])
    expect(root, "Invalid safetensors header length")


def test_tensor_load_errors(engine, tmp_path):
    root = make_checkpoint(tmp_path / "ckpt")
    r = run("--check-nvfp4-tensor", "--hf-model-dir", root, "--nvfp4-tensor", "model.language_model.layers.9.mlp.up_proj")
    assert r.returncode == 10 and "not found in model.safetensors.index.json" in r.stderr
    r = run("--check-nvfp4-tensor", "--hf-model-dir", tmp_path / "nowhere")
    assert r.returncode == 10 and "Model directory does not exist" in r.stderr


@pytest.mark.gpu
def test_check_and_bench_from_checkpoint(engine, oracle, tmp_path):
    """The tensor family read from disk gives the same projection as the arrays it was written from."""
    import torch

    base = "model.language_model.layers.0.mlp.gate_proj"
    fam, (codes, scales, s2) = family(base, 3584, 1024, seed=5, input_scale=0.5)
    root = tmp_path / "ckpt"
    root.mkdir()
    write_safetensors(root / "model.safetensors", fam)
    (root / "hf_quant_config.json").write_text(json.dumps(QUANT_CONFIG))
    r = run("--check-nvfp4-tensor", "--hf-model-dir", root, "--nvfp4-tensor", base, "--nvfp4-sample-rows", 32)
    assert r.returncode == 0, r.stderr
    assert "source_shape: [3584, 1024]" in r.stdout
    assert float(re.search(r"max_abs_error: ([-+0-9.eE]+)", r.stdout).group(1)) < 1e-6
    r = run("--bench-nvfp4-projection", "--hf-model-dir", root, "--nvfp4-projection-kernel", "b200-stream", "--bench-warmup", 2,
            "--bench-iters", 5)  # default tensor of the mode = layers.0.mlp.gate_proj
    assert r.returncode == 0, r.stderr
    assert float(re.search(r"max_abs_error: ([-+0-9.eE]+)", r.stdout).group(1)) < 2e-3
    del torch
