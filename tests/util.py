"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import moe_oracle as orc

H, I, E, TOPK = 6144, 768, 128, 4  # noqa: E741


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bf16_dev(bits):
    return dev(bits.view(np.int16)).view(torch.bfloat16)


def bits_of(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def atoms_to_rowmajor(atoms, bm):
    """scale atoms [blocks, n_atoms, 512] -> row-major scale bytes [blocks*bm, 4*n_atoms]."""
    nb, na, _ = atoms.shape
    r = np.arange(nb * bm)
    rr = r % bm
    out = np.zeros((nb * bm, na * 4), np.uint8)
    for c in range(na * 4):
        out[:, c] = atoms[r // bm, c // 4, (rr % 32) * 16 + (rr // 32) * 4 + (c % 4)]
    return out


def make_routing(tokens, kind, seed, experts=E):
    """ids int32 [T,4], weights fp32 [T,4]: the reference tests' routing kinds (tests/moe/.../workload.py:74-85,
    test_entry.py:32-40): uniform, hot (probability ~ rank^-1.2), four (experts 0..3), one (all pairs on one expert),
    dup (one expert in several slots of a token)."""
    rng = np.random.default_rng(seed)
    if kind == "hot":
        p = np.arange(1, experts + 1, dtype=np.float64) ** -1.2
        p /= p.sum()
        ids = np.stack([rng.choice(experts, TOPK, replace=False, p=p) for _ in range(tokens)])
    else:
        ids = np.stack([rng.permutation(experts)[:TOPK] for _ in range(tokens)])
    if kind == "four":
        ids = np.tile(np.arange(4), (tokens, 1))
    elif kind == "one":
        ids = np.full((tokens, TOPK), experts - 1)
    elif kind == "dup":
        ids[:, 1] = ids[:, 0]
    w = rng.random((tokens, TOPK)) + 0.5
    w = w / w.sum(1, keepdims=True) * 2.0
    return ids.astype(np.int32), w.astype(np.float32)


def oracle_slots(xq, xs, weights, ids, wts, tokens=None):
    """float32 slots [n, 4, H] of the chosen tokens from the CPU oracle."""
    sel = np.arange(xq.shape[0]) if tokens is None else np.asarray(tokens)
    _, slots = orc.w4a4_moe(xq[sel], xs[sel], *weights, wts[sel], ids[sel], return_slots=True)
    return slots


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / np.linalg.norm(b))
