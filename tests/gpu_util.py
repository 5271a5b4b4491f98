"""Helpers shared by the GPU parity tests (numpy <-> torch glue, seeded inputs, error measures)."""
import hashlib

import numpy as np
import torch


def cuda():
    return torch.device("cuda", 0)


def seeded_normal(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32) * scale


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def rel_fro(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    denom = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / (denom if denom > 0 else 1.0))


def np_of(t):
    return t.detach().float().cpu().numpy() if t.dtype != torch.int16 else t.detach().cpu().numpy()
