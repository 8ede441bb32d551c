"""On-disk formats next to the denoise path: the FP8 calibration cache and a synthetic checkpoint writer.

Calibration cache -- mirror of the reference's ``flash_rt/core/quant/calibrator.py:28-145``: static activation
scales are specific to a checkpoint and to the prefix length, so they are stored as JSON under a key made of a
fast checkpoint hash (SHA-256 of the first 64 KB of the file plus its size, 16 hex digits) and ``Se``, and
validated on load (version, hash, Se, count).  The record is NOT the reference's: it holds only the decoder table
(``ae_scales``, here one scale per (denoise step, layer, GEMM site), flattened in that order) and none of the
encoder fields, so a file of one implementation must never be taken for the other's.  The files therefore carry
their own suffix (``{hash}_Se{Se}.b200dec.json`` next to the reference's ``{hash}_Se{Se}.json``) and their own
``format`` tag; the reference neither finds nor overwrites them, and its files are left alone here.
Default location ``~/.flash_rt/calibration`` as in the reference; ``cache_dir`` overrides it.

Synthetic checkpoint -- a ``.safetensors`` file with the HF key names and shapes of the Pi0.5 action expert and
seeded random weights, so that ``load_model(path)`` can be exercised end to end without a trained checkpoint
(the reference reads the same keys, ``flash_rt/frontends/torch/pi05_rtx.py:118-292``).
"""
from __future__ import annotations

import hashlib
import json
import os
from pathlib import Path
from typing import Optional

CACHE_VERSION = 1
CACHE_FORMAT = "flashrt_b200.decoder_scales"      # distinguishes the record from the reference's calibration files
CACHE_SUFFIX = ".b200dec.json"
DEFAULT_CACHE_DIR = Path.home() / ".flash_rt" / "calibration"


def checkpoint_hash(checkpoint_path: str, read_bytes: int = 65536) -> str:
    p = Path(checkpoint_path)
    if p.is_dir():
        for name in ("model.safetensors", "model.safetensors.index.json"):
            if (p / name).exists():
                p = p / name
                break
        else:
            raise FileNotFoundError(f"No checkpoint file found in {checkpoint_path}")
    h = hashlib.sha256()
    with open(p, "rb") as f:
        h.update(f.read(read_bytes))
    h.update(str(p.stat().st_size).encode())
    return h.hexdigest()[:16]


def cache_path(ckpt_hash: str, Se: int, cache_dir=None) -> Path:
    return Path(cache_dir or DEFAULT_CACHE_DIR) / f"{ckpt_hash}_Se{Se}{CACHE_SUFFIX}"


def save_calibration(checkpoint_path: str, Se: int, ae_scales: list, metadata: Optional[dict] = None,
                     cache_dir=None) -> Path:
    ckpt = checkpoint_hash(checkpoint_path)
    path = cache_path(ckpt, Se, cache_dir)
    path.parent.mkdir(parents=True, exist_ok=True)
    data = {"format": CACHE_FORMAT, "version": CACHE_VERSION, "ckpt_hash": ckpt, "Se": int(Se), "num_ae_scales": len(ae_scales),
            "ae_scales": [float(v) for v in ae_scales]}
    if metadata is not None:
        data["metadata"] = metadata
    tmp = path.with_name(path.name + ".tmp")
    with open(tmp, "w") as f:
        json.dump(data, f, indent=2)
    os.replace(tmp, path)
    return path


def load_calibration(checkpoint_path: str, Se: int, expected_count: Optional[int] = None, cache_dir=None,
                     metadata: Optional[dict] = None) -> Optional[dict]:
    """The cached record, or None on any miss (no file, other version / checkpoint / Se / count / metadata)."""
    try:
        ckpt = checkpoint_hash(checkpoint_path)
    except (FileNotFoundError, IsADirectoryError):
        return None
    path = cache_path(ckpt, Se, cache_dir)
    if not path.exists():
        return None
    try:
        with open(path) as f:
            data = json.load(f)
    except (OSError, ValueError):
        return None
    if (data.get("format") != CACHE_FORMAT or data.get("version") != CACHE_VERSION or data.get("ckpt_hash") != ckpt
            or data.get("Se") != Se):
        return None
    scales = data.get("ae_scales")
    if not isinstance(scales, list) or data.get("num_ae_scales") != len(scales):
        return None
    if expected_count is not None and len(scales) != expected_count:
        return None
    if metadata is not None and data.get("metadata") != metadata:
        return None
    return data


def write_synthetic_checkpoint(path: str, seed: int = 0, layers: int = 18) -> str:
    """Write ``path`` (a ``.safetensors`` file, or a directory that receives ``model.safetensors``) with seeded
    random weights under the HF key names of the Pi0.5 action expert, stored in bf16."""
    import torch
    from safetensors.torch import save_file

    from .pi05_decoder import synthetic_state_dict
    p = Path(path)
    if p.suffix != ".safetensors":
        p.mkdir(parents=True, exist_ok=True)
        p = p / "model.safetensors"
    else:
        p.parent.mkdir(parents=True, exist_ok=True)
    sd = {k: v.to(torch.bfloat16).contiguous() for k, v in synthetic_state_dict(seed, layers).items()}
    save_file(sd, str(p), metadata={"format": "pt", "generator": f"flashrt_b200 synthetic seed={seed} layers={layers}"})
    return str(p)
