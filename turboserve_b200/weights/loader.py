"""Weights from safetensors, by tensor name.

A model folder holds ``config.json`` and either ``model.safetensors``, or shards listed in
``model.safetensors.index.json``, or any ``*.safetensors`` files
(``src/turboserve/engine/model/weights.py:137-178``). Every tensor the model declares is
looked up by its checkpoint name, checked for shape and copied to the device in the dtype
its role asks for: matrices in the compute dtype (bfloat16 when serving), biases and norm
gains in float32 (exact for values stored in bfloat16; a tensor stored in 32-bit stays so),
integer tables as int32. Nothing is loaded before everything has been checked, and one
:class:`WeightLoadError` lists all missing tensors, unexpected tensors and wrong shapes
(the reference is strict in the same way, ``weights.py:253-257,271-275``).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

SKIPPED_SUFFIXES = (".rotary_emb.inv_freq", ".attn.bias", ".attn.masked_bias", ".masked_bias")
INDEX_NAME = "model.safetensors.index.json"
SINGLE_NAME = "model.safetensors"
_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}


class WeightLoadError(RuntimeError):
    """The checkpoint cannot be loaded into the model; the message says everything that is wrong."""


def safetensors_files(model_dir: str | Path) -> list[Path]:
    folder = Path(model_dir)
    if folder.is_file():
        raise WeightLoadError(f"{folder} is a file; a model folder is needed")
    if not folder.is_dir():
        raise WeightLoadError(f"model folder {folder} does not exist")
    index = folder / INDEX_NAME
    if index.is_file():
        data = json.loads(index.read_text(encoding="utf-8"))
        weight_map = data.get("weight_map") if isinstance(data, dict) else None
        if not isinstance(weight_map, dict) or not weight_map:
            raise WeightLoadError(f"{index} has no 'weight_map'")
        files = []
        for name in sorted(set(weight_map.values())):
            path = folder / name
            if not path.is_file():
                raise WeightLoadError(f"{index} lists shard {name}, which is not in {folder}")
            files.append(path)
        return files
    single = folder / SINGLE_NAME
    if single.is_file():
        return [single]
    found = sorted(folder.glob("*.safetensors"))
    if found:
        return found
    if list(folder.glob("*.bin")) + list(folder.glob("*.pth")) + list(folder.glob("*.pt")):
        raise WeightLoadError(f"{folder} holds only pickled weights; safetensors are required")
    raise WeightLoadError(f"no safetensors file under {folder}")


def _read_header(path: Path) -> dict[str, tuple[tuple[int, ...], str]]:
    """Names, shapes and stored dtypes of a safetensors file, from its JSON header alone."""
    with open(path, "rb") as handle:
        raw = handle.read(8)
        if len(raw) != 8:
            raise WeightLoadError(f"{path} is not a safetensors file (too short)")
        size = int.from_bytes(raw, "little")
        if size <= 0 or size > 1 << 30:
            raise WeightLoadError(f"{path} is not a safetensors file (bad header length)")
        try:
            header = json.loads(handle.read(size).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise WeightLoadError(f"{path} is not a safetensors file: {exc}") from exc
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        out[name] = (tuple(int(s) for s in meta["shape"]), str(meta["dtype"]))
    return out


def map_name(stored: str, rewrites: tuple[tuple[str, str], ...] = ()) -> str:
    """The name the model knows a checkpoint tensor by: the first matching prefix is rewritten."""
    for old, new in rewrites:
        if stored.startswith(old):
            return new + stored[len(old):]
    return stored


def checkpoint_index(model_dir: str | Path, rewrites: tuple[tuple[str, str], ...] = ()) -> dict[str, tuple[Path, tuple[int, ...], str, str]]:
    """Every tensor of the checkpoint: name -> (file, shape, stored dtype, name in the file)."""
    index: dict[str, tuple[Path, tuple[int, ...], str, str]] = {}
    for path in safetensors_files(model_dir):
        for stored, (shape, dtype) in _read_header(path).items():
            if stored.endswith(SKIPPED_SUFFIXES):
                continue
            name = map_name(stored, rewrites)
            if name in index:
                raise WeightLoadError(f"tensor {name} is in both {index[name][0].name} and {path.name}")
            index[name] = (path, shape, dtype, stored)
    return index


def check_checkpoint(model, index: dict[str, tuple[Path, tuple[int, ...], str]]) -> None:
    """Raise one error that lists every missing, unexpected and wrongly shaped tensor."""
    expected = {p.name: p for p in model.named_params()}
    optional = model.optional_names()
    missing = sorted(name for name in expected if name not in index)
    unexpected = sorted(name for name in index if name not in expected and name not in optional)
    wrong = []
    for name, param in expected.items():
        if name in index and tuple(index[name][1]) != tuple(param.spec.shape):
            wrong.append(f"{name}: checkpoint has {list(index[name][1])}, model needs {list(param.spec.shape)}")
    if not (missing or unexpected or wrong):
        return
    lines = [f"checkpoint does not match {model.spec.architecture}:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(sorted(wrong)))
    raise WeightLoadError("\n".join(lines))


def load_weights(model, model_dir: str | Path) -> dict[str, str]:
    """Check the checkpoint against ``model`` and bind its tensors; returns name -> stored dtype."""
    from safetensors import safe_open

    index = checkpoint_index(model_dir, tuple(model.spec.names.prefix_rewrites))
    check_checkpoint(model, index)
    stored: dict[str, str] = {}
    handles: dict[Path, object] = {}

    def fetch(param) -> torch.Tensor:
        path, _, dtype, name_in_file = index[param.name]
        if path not in handles:
            handles[path] = safe_open(str(path), framework="pt", device="cpu")
        value = handles[path].get_tensor(name_in_file)
        stored[param.name] = dtype
        target = param.spec.device_dtype(model.dtype)
        if target == torch.int32 and value.dtype.is_floating_point:
            raise WeightLoadError(f"{param.name} is an integer table but is stored as {value.dtype}")
        return value.to(device=model.device, dtype=target)

    # part by part: a part's tensors go up, are fused by its bind() and dropped before the next
    # part's are read, so the device never holds much more than the model itself
    try:
        model.bind_stream(fetch)
    finally:
        for handle in handles.values():
            close = getattr(handle, "__exit__", None)
            if close is not None:
                close(None, None, None)
    return stored
