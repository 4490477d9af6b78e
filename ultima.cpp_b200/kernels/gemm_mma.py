"""Entry points of the tensor-core products over many small matrices (csrc/gemm_mma.cu): one matrix a head
(batched) and one matrix a tile of sorted rows (grouped, a routed feed-forward's experts)."""
from __future__ import annotations

import os

import torch

ENABLED = os.environ.get("ULTIMA_GEMM_MMA", "1") != "0"


def accepts_batched(a, w, out) -> bool:
    return False


def accepts_grouped(a, w, out, epilogue) -> bool:
    return False


def needs() -> list:
    """The libraries these products need on the bfloat16 path."""
    return []
