"""Shared helpers of the test-suite: raw-word <-> tensor conversion and golden loading."""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
TORCH_DT = {"fp16": torch.float16, "bf16": torch.bfloat16}


def to_tensor(words: np.ndarray, dtype: str, device="cpu") -> torch.Tensor:
    """uint16 words -> fp16/bf16 tensor with the same bits."""
    t = torch.from_numpy(np.ascontiguousarray(words).view(np.int16).copy())
    return t.to(device).view(TORCH_DT[dtype])


def to_words(t: torch.Tensor) -> np.ndarray:
    """fp16/bf16 tensor -> uint16 words (on the host)."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def load_npz(name: str):
    z = np.load(GOLDEN / f"{name}.npz")
    return {k: (str(z[k]) if k == "dtype" else z[k]) for k in z.files}


def load_json(name: str):
    return json.loads((GOLDEN / f"{name}.json").read_text())


FILL_CASES = ["fill_fp16_t8", "fill_bf16_t24", "fill_bf16_row1536"]
COPY_CASES = ["copy_fp16_fanout", "copy_bf16_l3"]
