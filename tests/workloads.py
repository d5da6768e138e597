"""Seeded synthetic inputs shared by the tests, the golden-vector generator and
the benchmark.  Everything is created on the CPU from ``torch.manual_seed`` so
that the same tensors can be rebuilt anywhere; callers move them to a device.

The full-size configurations are the five workloads of the benchmark spec:
  c1  rnnt_loss_simple            B=4   T=100 S=20  C=50
  c2  mutual_information_recursion B=32  S=128 T=512
  c3  pruned pipeline             B=64  T=500 S=100 C=500  D=512 s_range=5
  c4  unpruned rnnt_loss          B=8   T=200 S=50  C=500
  c5  pruned pipeline             B=512 T=400 S=60  C=5000 D=512 s_range=5
No public dataset is involved: i.i.d. normal activations, uniform symbols and
uniform lengths stand in for real encoder / decoder outputs.
"""
import math
import random

import torch


def _boundary(Sb, Tb):
    B = Sb.shape[0]
    z = torch.zeros(B, dtype=torch.int64)
    return torch.stack([z, z, Sb.to(torch.int64), Tb.to(torch.int64)], dim=1)


def reference_basic_tensors():
    """The fixed B=1,S=3,T=4,C=3 case of the reference's own unit test
    (fast_rnnt/python/tests/rnnt_loss_test.py:70-82)."""
    lm = torch.tensor([[[0, 0, 1], [0, 1, 1], [1, 0, 1], [2, 2, 0]]], dtype=torch.float)
    am = torch.tensor([[[0, 1, 2], [0, 0, 0], [0, 2, 4], [0, 3, 3]]], dtype=torch.float)
    symbols = torch.tensor([[0, 1, 0]], dtype=torch.long)
    return lm, am, symbols, 2


def config_c1():
    torch.manual_seed(0)
    B, T, S, C = 4, 100, 20, 50
    am = torch.randn(B, T, C)
    lm = torch.randn(B, S + 1, C)
    symbols = torch.randint(1, C, (B, S))
    Sb = torch.randint(10, 21, (B,))
    Tb = torch.randint(60, 101, (B,))
    return dict(am=am, lm=lm, symbols=symbols, boundary=_boundary(Sb, Tb), blank=0)


def config_c2(with_boundary: bool, B=32, S=128, T=512, seed=0):
    torch.manual_seed(seed)
    px = -6.0 * torch.rand(B, S, T + 1)
    py = -6.0 * torch.rand(B, S + 1, T)
    boundary = None
    if with_boundary:
        Sb = torch.randint(S // 2, S + 1, (B,))
        Tb = torch.stack([torch.randint(max(int(s), T // 2), T + 1, (1,))[0] for s in Sb])
        boundary = _boundary(Sb, Tb)
    return px, py, boundary


def config_c4(B=8, T=200, S=50, C=500, seed=0):
    torch.manual_seed(seed)
    logits = torch.randn(B, T, S + 1, C)
    symbols = torch.randint(1, C, (B, S))
    Sb = torch.randint(int(S * 0.6), S + 1, (B,))
    Tb = torch.randint(int(T * 0.75), T + 1, (B,))
    return dict(logits=logits, symbols=symbols, boundary=_boundary(Sb, Tb), blank=0)


PIPELINE_SIZES = {
    #        B    T    S    C     D   R   S_b range   T_b range
    "mini": (3, 40, 12, 20, 8, 4, (6, 12), (25, 40)),
    "small": (6, 90, 33, 70, 24, 5, (17, 33), (60, 90)),
    "c3": (64, 500, 100, 500, 512, 5, (50, 100), (350, 500)),
    "c5": (512, 400, 60, 5000, 512, 5, (30, 60), (280, 400)),
}


def pipeline_workload(name: str, rnnt_type: str = "regular", seed: int = 0, batch=None,
                      with_logit_inputs: bool = True):
    """Inputs of the full pruned pipeline (smoothed simple loss -> ranges ->
    pruning -> joiner -> pruned loss)."""
    B, T, S, C, D, R, (s_lo, s_hi), (t_lo, t_hi) = PIPELINE_SIZES[name]
    if batch is not None:
        B = batch
    torch.manual_seed(seed)
    am = 0.5 * torch.randn(B, T, C)
    lm = 0.5 * torch.randn(B, S + 1, C)
    symbols = torch.randint(1, C, (B, S))
    Sb = torch.randint(s_lo, s_hi + 1, (B,))
    Tb = torch.randint(t_lo, t_hi + 1, (B,))
    if rnnt_type != "regular":
        Tb = torch.maximum(Tb, Sb)
    enc = torch.randn(B, T, D)
    dec = torch.randn(B, S + 1, D)
    lin = torch.nn.Linear(D, C)  # default (Kaiming-uniform) init under the same seed
    small = name in ("mini", "small")
    return dict(am=am, lm=lm, symbols=symbols, boundary=_boundary(Sb, Tb), blank=0,
                enc=enc, dec=dec, joiner_w=lin.weight.detach().clone(),
                joiner_b=lin.bias.detach().clone(), s_range=R,
                lm_only_scale=0.25, am_only_scale=(0.1 if small else 0.0))


MI_SMALL_CASES = {
    "f32_regular_full": dict(dtype=torch.float32, modified=False, boundary="none", seed=1),
    "f32_regular_box": dict(dtype=torch.float32, modified=False, boundary="random", seed=2),
    "f32_modified_full": dict(dtype=torch.float32, modified=True, boundary="none", seed=3),
    "f32_modified_box": dict(dtype=torch.float32, modified=True, boundary="random", seed=4),
    "f64_regular_box": dict(dtype=torch.float64, modified=False, boundary="random", seed=5),
    "f64_modified_box": dict(dtype=torch.float64, modified=True, boundary="random", seed=6),
    "f32_regular_big": dict(dtype=torch.float32, modified=False, boundary="random", seed=7,
                            offset=15.0),
    "f32_regular_neginf": dict(dtype=torch.float32, modified=False, boundary="none", seed=8,
                               neg_inf_last=True),
    "f32_regular_wide": dict(dtype=torch.float32, modified=False, boundary="random", seed=9,
                             B=3, S=70, T=45),
}


def random_mi_boundary(B, S, T, modified, rng: random.Random, allow_empty=True):
    """Rows [s_begin,t_begin,s_end,t_end] with non-zero begins and (optionally)
    empty sequences, as in the reference's mutual_information_test.py:66-77."""
    rows = []
    for _ in range(B):
        this_S = rng.randint(0 if allow_empty else 1, S)
        this_T = rng.randint(this_S if modified else 1, T)
        s0 = rng.randint(0, S - this_S)
        t0 = rng.randint(0, T - this_T)
        rows.append([s0, t0, s0 + this_S, t0 + this_T])
    return torch.tensor(rows, dtype=torch.int64)


def mi_small(dtype=torch.float32, modified=False, boundary="none", seed=0, B=5, S=9, T=30,
             offset=0.0, neg_inf_last=False):
    torch.manual_seed(seed)
    rng = random.Random(seed)
    if modified and T < S:
        T = S + 3
    px = torch.randn(B, S, T + (0 if modified else 1), dtype=dtype) + offset
    py = torch.randn(B, S + 1, T, dtype=dtype) + offset
    if neg_inf_last and not modified:
        px[:, :, -1] = float("-inf")
    bnd = random_mi_boundary(B, S, T, modified, rng) if boundary == "random" else None
    return px, py, bnd


def joint_small(rnnt_type: str, seed=11):
    torch.manual_seed(seed)
    B, T, S, C = 3, 14, 6, 11
    logits = torch.randn(B, T, S + 1, C)
    symbols = torch.randint(0, C - 1, (B, S))
    Sb = torch.randint(2, S + 1, (B,))
    Tb = torch.randint(8, T + 1, (B,))
    return dict(logits=logits, symbols=symbols, boundary=_boundary(Sb, Tb), blank=C - 1)


def prune_edge_cases(seed=21):
    """Occupancy-like inputs for the prune-range edge cases: s_range > S, and
    tiny T with large S where the requested s_range must be raised."""
    out = {}
    torch.manual_seed(seed)
    # s_range > S (reference test at rnnt_loss_test.py:520-609)
    B, S, T = 2, 3, 20
    out["wide"] = dict(occ_x=torch.rand(B, S, T + 1), occ_y=torch.rand(B, S + 1, T),
                       boundary=_boundary(torch.tensor([3, 2]), torch.tensor([20, 17])),
                       s_range=7)
    # T tiny, S large (reference test at rnnt_loss_test.py:615-705)
    B, S, T = 2, 20, 4
    out["raise"] = dict(occ_x=torch.rand(B, S, T + 1), occ_y=torch.rand(B, S + 1, T),
                        boundary=_boundary(torch.tensor([20, 13]), torch.tensor([4, 3])),
                        s_range=3)
    # modified-shaped occupancies (px has T columns): window of the fix-up is 2
    B, S, T = 3, 9, 30
    out["modified"] = dict(occ_x=torch.rand(B, S, T), occ_y=torch.rand(B, S + 1, T),
                           boundary=_boundary(torch.tensor([9, 5, 7]), torch.tensor([30, 22, 9])),
                           s_range=3)
    return out


def lattice_cells(boundary, B, S, T):
    """Number of lattice cells inside the boundary boxes."""
    if boundary is None:
        return B * (S + 1) * (T + 1)
    b = boundary
    return int(((b[:, 2] - b[:, 0] + 1) * (b[:, 3] - b[:, 1] + 1)).sum().item())
