#!/usr/bin/env python
"""Benchmark of the pruned RNN-T loss hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c3|c5] [--no-stages] [--no-cpu-baseline]

One "step" is the whole pruned pipeline of the reference's documented usage,
forward and backward, on one batch of synthetic utterances:
  rnnt_loss_smoothed(return_grad) -> get_rnnt_prune_ranges -> do_rnnt_pruning ->
  joiner Linear(tanh(enc+dec)) -> rnnt_loss_pruned -> (simple+pruned).backward()
The joiner is the caller's network: by default this library's fused operator
rnnt_loss_pruned_joiner (fp16-pair tensor-core products, log-sum-exp in the epilogue), or
its pruned_joiner (--joiner tensorcore) or plain torch (--joiner torch); everything else
runs in libfrnnt_sm100.so.  Rank 0 prints ONE JSON line.

Under torchrun every rank works on its own batch (weak scaling; for --workload c5 the
global batch is built once from seed 0 and rank r takes its slice, so the all-reduced
loss does not depend on the number of ranks); the only collective is an NCCL all-reduce
of the scalar loss.

--impl reference times the reference's own python package on the host cores (its CPU
extension compiled into oracle/_ref, its python files installed under baseline/_ref by
__graft_entry__.build() where a checkout exists), or, where that install is absent,
the CPU oracle port of the same algorithm.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from tests import workloads  # noqa: E402  (seeded synthetic inputs)

L2_FLUSH_BYTES = 512 << 20
# all-reduced loss of the c5 global batch (B=512, seed 0), measured on one GPU
C5_GLOBAL_LOSS = 3130849.5

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the kernels
# the roofline lines name, workload c3, from the ncu captures summarised under profiles/
# (one small capture per kernel; the file names the command).  None: not captured.
NCU_TRAFFIC_C3 = {
    # profiles/kernels_c3_half_batch_ncu_full.txt: captured at half batch, doubled (every kernel
    # streams its operands once, so its traffic grows with the number of rows)
    "fused_fwd_product": 2 * 277.7e6, "fused_bwd_grad_input": 2 * 462.3e6,
    "fused_bwd_grad_weight": 2 * 331.5e6,
    "mi_forward": 2 * 8.3e6, "mi_backward": 2 * 5.9e6, "mi_forward_pruned": 2 * 8.3e6,
    "mi_backward_pruned": 2 * 5.9e6,
}


def measured_tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timing runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------
# the step
# ------------------------------------------------------------------------------
def make_step(fr, wl, joiner="torch", overlap=False):
    """Returns step(inputs) -> loss for the pruned pipeline; `fr` is the loss package
    (ours on CUDA, or the CPU oracle / the reference wrapped to the same names).
    joiner: how the caller's network between pruning and the pruned loss runs --
      "torch"       do_rnnt_pruning + torch Linear(tanh(.)) + rnnt_loss_pruned (the
                    reference's documented usage, the only form the reference offers),
      "tensorcore"  this library's pruned_joiner (3xTF32 products) + rnnt_loss_pruned,
      "fused"       this library's rnnt_loss_pruned_joiner: one operator from enc / dec to
                    the pruned lattices (fp16-pair products, log-sum-exp in the epilogue).
    overlap: run the simple loss on a second CUDA stream (see inside)."""
    blank, R = wl["blank"], wl["s_range"]
    ls, as_ = wl["lm_only_scale"], wl["am_only_scale"]
    side = [None]   # CUDA only: the stream the simple loss runs on

    def step(t):
        on_gpu = t["am"].is_cuda
        if on_gpu and overlap:
            # The simple loss runs on a second stream.  Forward nothing is gained (the prune
            # ranges need its occupancies), but autograd runs every backward node on the stream
            # of its forward: the simple loss's backward (small kernels + short products) then
            # overlaps with the pruned branch's large products instead of queueing behind them.
            if side[0] is None:
                side[0] = torch.cuda.Stream(device=t["am"].device)
            main = torch.cuda.current_stream(t["am"].device)
            side[0].wait_stream(main)
            ctx = torch.cuda.stream(side[0])
        else:
            import contextlib
            main, ctx = None, contextlib.nullcontext()
        am = t["am"].requires_grad_(True)
        lm = t["lm"].requires_grad_(True)
        enc = t["enc"].requires_grad_(True)
        dec = t["dec"].requires_grad_(True)
        W = t["joiner_w"].requires_grad_(True)
        bias = t["joiner_b"].requires_grad_(True)
        for x in (am, lm, enc, dec, W, bias):
            x.grad = None
        with ctx:
            simple, (gx, gy) = fr.rnnt_loss_smoothed(
                lm=lm, am=am, symbols=t["symbols"], termination_symbol=blank, lm_only_scale=ls,
                am_only_scale=as_, boundary=t["boundary"], reduction="sum", return_grad=True)
        if main is not None:
            main.wait_stream(side[0])
        ranges = fr.get_rnnt_prune_ranges(px_grad=gx, py_grad=gy, boundary=t["boundary"], s_range=R)
        if joiner == "fused":
            pruned = fr.rnnt_loss_pruned_joiner(
                am=enc, lm=dec, ranges=ranges, joiner_weight=W, joiner_bias=bias,
                symbols=t["symbols"], termination_symbol=blank, boundary=t["boundary"],
                reduction="sum")
        else:
            if joiner == "tensorcore":
                logits = fr.pruned_joiner(enc, dec, ranges, W, bias)
            else:
                am_p, lm_p = fr.do_rnnt_pruning(am=enc, lm=dec, ranges=ranges)
                logits = torch.nn.functional.linear(torch.tanh(am_p + lm_p), W, bias)
            pruned = fr.rnnt_loss_pruned(logits=logits, symbols=t["symbols"], ranges=ranges,
                                         termination_symbol=blank, boundary=t["boundary"],
                                         reduction="sum")
        loss = simple + pruned
        loss.backward()
        if main is not None:
            main.wait_stream(side[0])   # the step ends when both branches have
        return loss.detach()

    return step


class OracleApi:
    """The CPU oracle under the reference's function names (CPU baseline only)."""

    def __init__(self):
        from oracle import rnnt_oracle as orc
        self.orc = orc

    def rnnt_loss_smoothed(self, lm, am, symbols, termination_symbol, lm_only_scale,
                           am_only_scale, boundary, reduction, return_grad):
        return self.orc.loss_smoothed(lm, am, symbols, termination_symbol, lm_only_scale,
                                      am_only_scale, boundary, "regular", 0.0, reduction,
                                      return_grad)

    def get_rnnt_prune_ranges(self, px_grad, py_grad, boundary, s_range):
        return self.orc.prune_ranges(px_grad, py_grad, boundary, s_range)

    def do_rnnt_pruning(self, am, lm, ranges):
        return self.orc.prune(am, lm, ranges)

    def rnnt_loss_pruned(self, logits, symbols, ranges, termination_symbol, boundary, reduction):
        return self.orc.loss_pruned(logits, symbols, ranges, termination_symbol, boundary,
                                    "regular", 0.0, reduction)


TENSOR_KEYS = ("am", "lm", "enc", "dec", "joiner_w", "joiner_b", "symbols", "boundary")

_REFERENCE = None


def load_reference_package():
    """The reference's own python package, if it was installed next to this file:
    baseline/_ref/fast_rnnt (its python files) on one of its compiled extensions --
    oracle/_ref/cuda/_fast_rnnt.so (CPU + CUDA kernels) or oracle/_ref/_fast_rnnt.so (CPU).
    Returns (module, has_cuda_kernels) or None."""
    global _REFERENCE
    if _REFERENCE is not None:
        return _REFERENCE or None
    _REFERENCE = False
    pkg = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(pkg, "fast_rnnt", "__init__.py")):
        return None
    for d in (os.path.join(ROOT, "oracle", "_ref", "cuda"), os.path.join(ROOT, "oracle", "_ref")):
        if os.path.exists(os.path.join(d, "_fast_rnnt.so")):
            sys.path.insert(0, d)
            sys.path.insert(0, pkg)
            try:
                import _fast_rnnt  # noqa: F401  (the package imports it by this name)
                import fast_rnnt
                _REFERENCE = (fast_rnnt, bool(_fast_rnnt.with_cuda()))
                return _REFERENCE
            except Exception as e:  # pragma: no cover
                print(f"reference package not importable from {d}: {e}", file=sys.stderr)
                sys.path.remove(d)
                sys.path.remove(pkg)
    return None


def cpu_reference_run(workload, sample_batch, steps, warmup):
    """Times the reference's CPU implementation on the host cores: its own package where
    installed (kind "reference"), else the CPU oracle port (kind "port").  Returns
    (utt/s, ms per step, kind, loss of the sample)."""
    wl = workloads.pipeline_workload(workload, batch=sample_batch)
    ref = load_reference_package()
    api, kind = (ref[0], "reference") if ref else (OracleApi(), "port")
    step = make_step(api, wl)
    t = {k: wl[k].clone() for k in TENSOR_KEYS}
    for _ in range(warmup):
        step(t)
    times, loss = [], None
    for _ in range(steps):
        t0 = time.perf_counter()
        loss = step(t)
        times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    grads = {k: t[k].grad.detach().clone() for k in ("am", "lm", "enc", "dec", "joiner_w")}
    return sample_batch / sec, sec * 1e3, kind, float(loss), grads


def reference_cuda_run(workload, batch, sample_batch, cpu_grads, dev):
    """The reference's own pipeline on the GPU (its torch ops on device tensors + its CUDA
    mutual-information kernels), device-timed, and -- on the CPU leg's sample -- the
    reference's own CPU <-> CUDA gradient gap: the noise floor of any comparison."""
    ref = load_reference_package()
    if not ref or not ref[1]:
        return None, None
    api = ref[0]
    wl = workloads.pipeline_workload(workload, batch=batch)
    step = make_step(api, wl)
    t = {k: wl[k].to(dev) for k in TENSOR_KEYS}
    for _ in range(2):
        step(t)
    torch.cuda.synchronize()
    ms = []
    for _ in range(5):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        step(t)
        e.record()
        e.synchronize()
        ms.append(s.elapsed_time(e))
    med = statistics.median(ms)
    out = {"ms_per_step": round(med, 3), "value": round(batch / (med * 1e-3), 1), "unit": "utt/s",
           "what": "the reference's python package on CUDA tensors with its own CUDA kernels, "
                   "joiner in torch (cuBLAS fp32), same workload, CUDA events, median of 5; one "
                   "stream (its kernels launch on the legacy default stream)"}
    noise = None
    if cpu_grads is not None:
        wl_s = workloads.pipeline_workload(workload, batch=sample_batch)
        ts = {k: wl_s[k].to(dev) for k in TENSOR_KEYS}
        make_step(api, wl_s)(ts)
        noise = {k: float((ts[k].grad.cpu() - cpu_grads[k]).abs().max()) for k in cpu_grads}
        noise["what"] = (f"max |gradient on CPU - gradient on CUDA| of the reference itself, "
                         f"{sample_batch} utterances")
    return out, noise


# ------------------------------------------------------------------------------
# per-stage timing (each C-ABI stage alone, CUDA events, L2 flushed in between)
# ------------------------------------------------------------------------------
def time_call(fn, flush, reps=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(reps):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        ms.append(s.elapsed_time(e))
    return statistics.median(ms)


def stage_table(fr, wl, dev, flush, hbm_gbs):
    """Times every stage of the loss path alone and relates it to its
    algorithmic bytes (each input read once, each output written once)."""
    from fast_rnnt_b200 import mutual_information as mi
    t = {k: wl[k].to(dev) for k in TENSOR_KEYS}
    B, T, C = t["am"].shape
    S = t["lm"].shape[1] - 1
    D = t["enc"].shape[2]
    R = wl["s_range"]
    ls, as_ = wl["lm_only_scale"], wl["am_only_scale"]
    es = 4
    cells_box = workloads.lattice_cells(wl["boundary"], B, S, T)
    lat = es * B * (S * (T + 1) + (S + 1) * T)

    lm = t["lm"].clone().requires_grad_(True)
    am = t["am"].clone().requires_grad_(True)
    px, py = fr.get_rnnt_logprobs_smoothed(lm=lm, am=am, symbols=t["symbols"],
                                           termination_symbol=0, lm_only_scale=ls,
                                           am_only_scale=as_, boundary=t["boundary"])
    gpx, gpy = torch.rand_like(px), torch.rand_like(py)
    pxd, pyd = px.detach(), py.detach()
    _, _, branch = mi.mi_forward(pxd, pyd, t["boundary"])
    ones = torch.ones(B, device=dev)
    ox, oy = mi.mi_backward_from_lattice(pxd, branch, t["boundary"], ones, py.shape)
    ranges = fr.get_rnnt_prune_ranges(px_grad=ox, py_grad=oy, boundary=t["boundary"], s_range=R)
    dec = t["dec"].clone().requires_grad_(True)
    _, lm_p = fr.do_rnnt_pruning(am=t["enc"], lm=dec, ranges=ranges)
    g_lm_p = torch.rand_like(lm_p)
    logits = torch.randn(B, T, R, C, device=dev).requires_grad_(True)
    ppx, ppy = fr.get_rnnt_logprobs_pruned(logits=logits, symbols=t["symbols"], ranges=ranges,
                                           termination_symbol=0, boundary=t["boundary"])
    ppxd, ppyd = ppx.detach(), ppy.detach()
    _, _, pbranch = mi.mi_forward(ppxd, ppyd, t["boundary"])

    def fwd_simple():
        fr.get_rnnt_logprobs_smoothed(lm=t["lm"], am=t["am"], symbols=t["symbols"],
                                      termination_symbol=0, lm_only_scale=ls, am_only_scale=as_,
                                      boundary=t["boundary"])

    stages = [
        # name, callable, algorithmic bytes, flops (for the contraction) or None
        ("simple_logprobs_fwd", fwd_simple, es * B * (T + S + 1) * C + lat, 2.0 * B * (S + 1) * T * C),
        ("simple_logprobs_bwd",
         lambda: torch.autograd.grad((px, py), (lm, am), (gpx, gpy), retain_graph=True),
         2 * es * B * (T + S + 1) * C + lat, 4.0 * B * (S + 1) * T * C),
        ("mi_forward", lambda: mi.mi_forward(pxd, pyd, t["boundary"]), 12 * cells_box, None),
        ("mi_backward", lambda: mi.mi_backward_from_lattice(pxd, branch, t["boundary"], ones,
                                                            py.shape), 8 * cells_box + lat, None),
        ("mi_forward_pruned", lambda: mi.mi_forward(ppxd, ppyd, t["boundary"]), 12 * cells_box, None),
        ("mi_backward_pruned", lambda: mi.mi_backward_from_lattice(ppxd, pbranch, t["boundary"],
                                                                   ones, py.shape),
         8 * cells_box + lat, None),
        ("prune_ranges", lambda: fr.get_rnnt_prune_ranges(px_grad=ox, py_grad=oy,
                                                          boundary=t["boundary"], s_range=R),
         lat + 8 * B * T * R, None),
        ("prune_gather_fwd", lambda: fr.do_rnnt_pruning(am=t["enc"], lm=t["dec"], ranges=ranges),
         es * B * T * R * D + es * B * (S + 1) * D + 8 * B * T * R, None),
        ("prune_gather_bwd", lambda: torch.autograd.grad(lm_p, dec, g_lm_p, retain_graph=True),
         es * B * T * R * D + es * B * (S + 1) * D, None),
        ("lsm_gather_fwd", lambda: fr.get_rnnt_logprobs_pruned(
            logits=logits.detach(), symbols=t["symbols"], ranges=ranges, termination_symbol=0,
            boundary=t["boundary"]), es * B * T * R * C + lat + 3 * es * B * T * R, None),
        ("lsm_gather_bwd", lambda: torch.autograd.grad((ppx, ppy), logits, (gpx, gpy),
                                                       retain_graph=True),
         2 * es * B * T * R * C, None),
    ]
    # the joiner's kernels (harness around the loss path, but most of a step's time): the
    # same calls fast_rnnt_b200.pruned_joiner makes, one at a time
    import importlib
    from fast_rnnt_b200 import _lib
    flin = importlib.import_module("fast_rnnt_b200.linear")   # the package exports a function of that name
    M = B * T * R
    W = t["joiner_w"].contiguous()
    Wt = W.t().contiguous()
    act = torch.empty(B, T, R, D, device=dev)
    gz = torch.randn(M, D, device=dev)
    g_logits = torch.randn(M, C, device=dev)
    enc_g, dec_g = torch.empty(B, T, D, device=dev), torch.empty(B, S + 1, D, device=dev)
    jscratch = torch.empty(max(1, _lib.lib().frnnt_joiner_input_grads_scratch_bytes(B, T, D)),
                           dtype=torch.uint8, device=dev)
    sp = _lib.stream_ptr(dev)

    def j_tanh():
        _lib.call("frnnt_pruned_tanh", 0, _lib.ptr(t["enc"]), _lib.ptr(t["dec"]), _lib.ptr(ranges),
                  _lib.ptr(act), B, S + 1, T, R, D, sp)

    j_tanh()
    act2 = act.reshape(M, D)
    gemm_flops = 2.0 * M * C * D
    stages += [
        ("joiner_tanh", j_tanh, es * M * D + es * B * (T + S + 1) * D + 8 * M, None),
        ("joiner_linear_fwd", lambda: flin._matmul_nt(act2, W, t["joiner_b"], M, C, D),
         es * (M * D + M * C + C * D), gemm_flops),
        ("joiner_linear_grad_input", lambda: flin._matmul_nt(g_logits, Wt, None, M, D, C, tanh_out=act2),
         es * (M * C + 2 * M * D + C * D), gemm_flops),
        ("joiner_linear_grad_weight", lambda: flin._matmul_tn(g_logits, act2, C, D, M, want_colsum=True),
         es * (M * C + M * D + C * D), gemm_flops),
        ("joiner_input_grads", lambda: _lib.call(
            "frnnt_joiner_input_grads", _lib.ptr(gz), _lib.ptr(ranges), _lib.ptr(enc_g),
            _lib.ptr(dec_g), _lib.ptr(jscratch), B, S + 1, T, R, D, sp),
         es * (M * D + B * (T + S + 1) * D), None),
    ]
    # the fused operator (--joiner fused): as a whole, and its three products alone on the
    # fp16-pair engine (planes made from the same random matrices)
    lib = _lib.lib()
    sym, bnd = t["symbols"], t["boundary"]
    S1 = S + 1
    pj_saved = torch.empty(max(1, lib.frnnt_pruned_joiner_saved_bytes(B, T, R, S, C, D)),
                           dtype=torch.uint8, device=dev)
    pj_fs = torch.empty(max(1, lib.frnnt_pruned_joiner_forward_scratch_bytes(B, T, R, S, C, D)),
                        dtype=torch.uint8, device=dev)
    pj_bs = torch.empty(max(1, lib.frnnt_pruned_joiner_backward_scratch_bytes(B, T, R, S, C, D)),
                        dtype=torch.uint8, device=dev)
    w_g, b_g = torch.empty(C, D, device=dev), torch.empty(C, device=dev)

    def pj_fwd():
        _lib.call("frnnt_pruned_joiner_logprobs_forward", 0, _lib.ptr(t["enc"]), _lib.ptr(t["dec"]),
                  _lib.ptr(ranges), _lib.ptr(W), _lib.ptr(t["joiner_b"]), _lib.ptr(sym), _lib.ptr(bnd),
                  _lib.ptr(ppxd), _lib.ptr(ppyd), _lib.ptr(pj_saved), _lib.ptr(pj_fs), B, T, R, S, C, D,
                  0, 0, ctypes.c_double(0.0), sp)

    def pj_bwd():
        _lib.call("frnnt_pruned_joiner_logprobs_backward", _lib.ptr(gpx), _lib.ptr(gpy), _lib.ptr(ranges),
                  _lib.ptr(sym), _lib.ptr(bnd), _lib.ptr(pj_saved), _lib.ptr(pj_bs), _lib.ptr(enc_g),
                  _lib.ptr(dec_g), _lib.ptr(w_g), _lib.ptr(b_g), B, T, R, S, C, D, 0, 0, sp)

    Cp = (C + 63) // 64 * 64

    def fwd_part(part):
        return lambda: _lib.call(
            "frnnt_pruned_joiner_logprobs_forward_part", part, _lib.ptr(t["enc"]), _lib.ptr(t["dec"]),
            _lib.ptr(ranges), _lib.ptr(W), _lib.ptr(t["joiner_b"]), _lib.ptr(sym), _lib.ptr(bnd),
            _lib.ptr(ppxd), _lib.ptr(ppyd), _lib.ptr(pj_saved), _lib.ptr(pj_fs), B, T, R, S, C, D, 0, 0, sp)

    def bwd_part(part):
        return lambda: _lib.call(
            "frnnt_pruned_joiner_logprobs_backward_part", part, _lib.ptr(gpx), _lib.ptr(gpy),
            _lib.ptr(ranges), _lib.ptr(sym), _lib.ptr(bnd), _lib.ptr(pj_saved), _lib.ptr(pj_bs),
            _lib.ptr(enc_g), _lib.ptr(dec_g), _lib.ptr(w_g), _lib.ptr(b_g), B, T, R, S, C, D, 0, 0, sp)

    pj_fwd()
    pj_bwd()   # every buffer the parts below work on is filled
    planes_bytes = es * (B * (T + S1) * D + M * D + 3 * C * D) + 8 * M
    stages += [
        ("fused_joiner_lattices_fwd", pj_fwd,
         es * (B * (T + S1) * D + 8 * M // 4 + M * D + M * C + C * D) + lat, gemm_flops),
        ("fused_joiner_lattices_bwd", pj_bwd,
         lat + es * (2 * M * C + 2 * M * D + B * (T + S1) * D + 2 * C * D), 2 * gemm_flops),
        # the same calls, one part at a time (what a step launches, kernel group by kernel group)
        ("fused_fwd_planes", fwd_part(0), planes_bytes, None),
        ("fused_fwd_product", fwd_part(1), es * (M * D + M * C + C * D), gemm_flops),
        ("fused_fwd_lattices", fwd_part(2), lat + 8 * M * 3 + es * M * (C // 128 + 1) * 2, None),
        ("fused_bwd_planes", bwd_part(0), lat + es * M * (C + Cp), None),
        ("fused_bwd_grad_input", bwd_part(1), es * (M * Cp + 2 * M * D + C * D), gemm_flops),
        ("fused_bwd_input_grads", bwd_part(4), es * (M * D + B * (T + S1) * D), None),
        ("fused_bwd_grad_weight", bwd_part(3), es * (M * Cp + M * D + C * D), gemm_flops),
    ]
    out = {}
    for name, fn, nbytes, flops in stages:
        ms = time_call(fn, flush)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": round(ms, 4), "alg_bytes": int(nbytes), "gbs": round(gbs, 1),
                     "hbm_frac": round(gbs / hbm_gbs, 4)}
        if flops:
            out[name]["tflops"] = round(flops / (ms * 1e-3) / 1e12, 2)
    return out, cells_box


COMMON_STAGES = ["simple_logprobs_fwd", "simple_logprobs_bwd", "mi_forward", "mi_backward",
                 "mi_forward_pruned", "mi_backward_pruned", "prune_ranges"]
STEP_STAGES = {
    # stages of the table above that one timed step launches, by --joiner
    "fused": COMMON_STAGES + ["fused_fwd_planes", "fused_fwd_product", "fused_fwd_lattices", "fused_bwd_planes",
                              "fused_bwd_grad_input", "fused_bwd_input_grads", "fused_bwd_grad_weight"],
    "tensorcore": COMMON_STAGES + ["joiner_tanh", "joiner_linear_fwd", "lsm_gather_fwd", "lsm_gather_bwd",
                                   "joiner_linear_grad_input", "joiner_linear_grad_weight",
                                   "joiner_input_grads"],
    "torch": COMMON_STAGES + ["prune_gather_fwd", "lsm_gather_fwd", "lsm_gather_bwd", "prune_gather_bwd"],
}
PRODUCT_STAGES = {"fused": ["fused_fwd_product", "fused_bwd_grad_input", "fused_bwd_grad_weight"],
                  "tensorcore": ["joiner_linear_fwd", "joiner_linear_grad_input",
                                 "joiner_linear_grad_weight"],
                  "torch": []}


def mi_c2_table(dev, flush):
    """The standalone recursion on the configuration the metric names for it (B=32,
    S=128, T=512, log-probs uniform on (-6, 0)): lattice cells per second, forward alone
    and forward + backward (what return_grad costs), without and with boundaries."""
    from fast_rnnt_b200 import mutual_information as mi
    out = {}
    for tag, with_boundary in (("full", False), ("bounded", True)):
        px, py, bnd = workloads.config_c2(with_boundary)
        B, S, _ = px.shape
        T = py.shape[2]
        px, py = px.to(dev), py.to(dev)
        cells = workloads.lattice_cells(bnd, B, S, T) if bnd is not None else B * (S + 1) * (T + 1)
        bnd = bnd.to(dev) if bnd is not None else None
        ones = torch.ones(B, device=dev)

        def fwd():
            return mi.mi_forward(px, py, bnd)

        def fwd_bwd():
            _, _, lat = mi.mi_forward(px, py, bnd)
            mi.mi_backward_from_lattice(px, lat, bnd, ones, py.shape)

        f_ms, fb_ms = time_call(fwd, flush), time_call(fwd_bwd, flush)
        out[tag] = {"cells": int(cells), "fwd_ms": round(f_ms, 4), "fwd_bwd_ms": round(fb_ms, 4),
                    "cells_per_s_fwd": round(cells / (f_ms * 1e-3), 1),
                    "cells_per_s_fwd_bwd": round(cells / (fb_ms * 1e-3), 1)}
    return out


# ------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=["c3", "c5", "small"])
    ap.add_argument("--batch", type=int, default=None, help="utterances per GPU")
    ap.add_argument("--joiner", default="fused", choices=["fused", "tensorcore", "torch"],
                    help="the caller's joiner: this library's fused rnnt_loss_pruned_joiner "
                         "(fp16-pair tcgen05 products), its pruned_joiner (3xTF32 products), or "
                         "torch.nn.functional.linear (cuBLAS fp32)")
    ap.add_argument("--no-overlap", action="store_true",
                    help="keep the simple loss on the main stream (its backward then queues behind "
                         "the pruned branch's instead of overlapping with it)")
    ap.add_argument("--no-graph", action="store_true",
                    help="enqueue every step eagerly instead of replaying a CUDA graph of it")
    ap.add_argument("--input-dtype", default="f32", choices=["f32", "bf16", "f16"],
                    help="f32: the benchmark.  bf16 / f16: the same step on 16-bit am / lm / enc / dec "
                         "(float32 arithmetic); reported with that label, stages and CPU legs skipped")
    ap.add_argument("--no-stages", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    sizes = workloads.PIPELINE_SIZES[args.workload]
    batch = args.batch or (sizes[0] if args.workload != "c5" else sizes[0] // world)
    cfg = {"workload": f"{args.workload}: pruned RNN-T loss pipeline fwd+bwd (smoothed simple loss, "
                       f"prune ranges, pruning, joiner, pruned loss)",
           "B_per_gpu": batch, "T": sizes[1], "S": sizes[2], "C": sizes[3], "D": sizes[4],
           "s_range": sizes[5], "global_batch": batch * world,
           "parallelism": f"batch sharded over {world} GPU(s), scalar-loss all-reduce",
           "joiner": f"Linear({sizes[4]}->{sizes[3]})(tanh(enc_pruned + dec_pruned)), float32 results",
           "l2": f"value and stages: flushed between timed steps ({L2_FLUSH_BYTES >> 20} MiB write); e2e: "
                 "every step's inputs are a fresh upload larger than L2",
           "e2e_upload": "all inputs of a step collated in one page-locked (cudaHostRegister) buffer, "
                         "one H2D copy per step on a copy stream that runs one step ahead"}

    joiner_impl = {"fused": "fast_rnnt_b200.rnnt_loss_pruned_joiner: one operator from enc / dec to the "
                            "pruned lattices, fp16-pair tcgen05 products (fp32-level accuracy), "
                            "log-sum-exp in the forward product's epilogue",
                   "tensorcore": "fast_rnnt_b200.pruned_joiner (gather+add+tanh kernel, 3xTF32 tcgen05 "
                                 "products) + rnnt_loss_pruned",
                   "torch": "do_rnnt_pruning + torch Linear(tanh(.)) (cuBLAS fp32) + rnnt_loss_pruned"}

    # -------------------------------------------------------------- reference arm
    if args.impl == "reference":
        if rank != 0:
            return
        torch.set_num_threads(os.cpu_count() or 1)
        sample = min(batch, 16)
        value, ms, kind, _, _ = cpu_reference_run(args.workload, sample, max(1, args.steps), args.warmup)
        cores = torch.get_num_threads()
        what = ("the reference's own python package on its CPU extension" if kind == "reference"
                else "CPU oracle port: torch CPU ops + C recursion")
        line = {"impl": "reference", "metric": "utterances/sec", "value": round(value, 3),
                "unit": "utt/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
                "joiner_impl": "do_rnnt_pruning + torch Linear(tanh(.)) on the CPU + rnnt_loss_pruned",
                "cpu_baseline": {"value": round(value, 3), "unit": "utt/s", "cores": cores,
                                 "kind": kind,
                                 "sample": f"{sample} utterances of the {args.workload} batch per step "
                                           f"({what})"},
                "e2e": {"value": round(value, 3), "unit": "utt/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    # ----------------------------------------------------------------------- ours
    import fast_rnnt_b200 as fr
    from fast_rnnt_b200 import _lib
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.lib()
    lib.frnnt_launch_count.restype = __import__("ctypes").c_longlong

    if args.workload == "c5" and args.batch is None:
        # one global batch from seed 0, rank r takes rows [r*B/n, (r+1)*B/n): the all-reduced
        # loss is then the same number at every n
        from fast_rnnt_b200 import sharding
        full = workloads.pipeline_workload("c5", batch=sizes[0], seed=0)
        wl = sharding.shard_batch(full, [k for k in TENSOR_KEYS if k not in ("joiner_w", "joiner_b")],
                                  rank, world)
        del full
    else:
        wl = workloads.pipeline_workload(args.workload, batch=batch, seed=rank)
    if args.input_dtype != "f32":
        # NOT the benchmark's configuration (the reference takes float32): am / lm / enc / dec as
        # 16-bit tensors, read by the kernels directly, all arithmetic still float32
        half = torch.bfloat16 if args.input_dtype == "bf16" else torch.float16
        for k in ("am", "lm", "enc", "dec"):
            wl[k] = wl[k].to(half)
    host = {k: wl[k].pin_memory() for k in TENSOR_KEYS}
    resident = {k: v.to(dev) for k, v in host.items()}
    inner = make_step(fr, wl, args.joiner, overlap=not args.no_overlap)

    from fast_rnnt_b200 import sharding

    last_loss = [None]
    # One CUDA graph per set of input buffers (the resident ones, and the two upload buffers
    # of the e2e loop), captured at the first call, i.e. during warm-up; they share one pool.
    graphs, pool = {}, (None if args.no_graph else torch.cuda.graph_pool_handle())

    graph_note = [None]

    def step(t, key="resident"):
        if not args.no_graph and key not in graphs:
            from fast_rnnt_b200.graphs import GraphedStep
            try:
                graphs[key] = GraphedStep(inner, t, pool=pool)
            except Exception as e:  # the harness goes on eagerly, and says so in its line
                args.no_graph = True
                graphs.clear()
                graph_note[0] = f"off: capture failed ({type(e).__name__}: {str(e)[:200]})"
                print("bench: CUDA graph capture failed, running eagerly:", e, file=sys.stderr)
                torch.cuda.synchronize()
        if args.no_graph:
            loss = inner(t)
        else:
            loss = graphs[key]()
        last_loss[0] = sharding.allreduce_loss(loss)
        return last_loss[0]

    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(run_one, steps, warmup):
        for _ in range(warmup):
            run_one()
        barrier()
        pairs = []
        for _ in range(steps):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            run_one()
            e.record()
            pairs.append((s, e))
        barrier()
        total_ms = sum(s.elapsed_time(e) for s, e in pairs)
        if world > 1:
            tt = torch.tensor([total_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            total_ms = float(tt.item())
        return total_ms

    # value: inputs resident in HBM
    with ClockSampler(local_rank) as clocks:
        n0 = lib.frnnt_launch_count()
        total_ms = timed(lambda: step(resident), args.steps, args.warmup)
        launches = (graphs["resident"].launches if graphs else
                    (lib.frnnt_launch_count() - n0) // (args.steps + args.warmup))
    ms_per_step = total_ms / args.steps
    value = batch * world / (ms_per_step * 1e-3)

    # e2e: host (pinned) inputs, H2D of every input and D2H of the loss inside the timed region
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()
    io_keys = ("am", "lm", "enc", "dec", "symbols", "boundary")

    # A training loop uploads the next batch while the current one is computed: a copy
    # stream runs one step ahead.  The batch is collated the way a data loader does it,
    # into ONE pinned staging buffer (the host tensors are views of it), and goes up as
    # one copy: on these boxes every cudaMemcpyAsync carries ~0.6 ms of fixed cost, which
    # six separate tensors would pay six times.  Every step's upload, its compute and the
    # read-back of its loss are inside the timed region; the first upload is not hidden.
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    offsets, total = {}, 0
    for k in io_keys:
        offsets[k] = total
        total += (host[k].numel() * host[k].element_size() + 255) // 256 * 256
    # page-locked with cudaHostRegister: on these boxes a buffer from torch's pin_memory()
    # uploads at 38 GB/s, a registered (or cudaHostAlloc'ed) one at 55 GB/s
    staging = torch.empty(total, dtype=torch.uint8)
    try:
        registered = int(torch.cuda.cudart().cudaHostRegister(staging.data_ptr(), total, 0)) == 0
    except Exception:
        registered = False
    if not registered or not staging.is_pinned():
        staging = staging.pin_memory()

    def view_of(buf, k):
        n = host[k].numel() * host[k].element_size()
        return buf[offsets[k]:offsets[k] + n].view(host[k].dtype).view(host[k].shape)

    for k in io_keys:
        view_of(staging, k).copy_(host[k])
    host_rows = host["boundary"].tolist() if hasattr(fr, "provide_boundary_rows") else None
    dev_bufs = [torch.empty(total, dtype=torch.uint8, device=dev) for _ in range(2)]
    free_ev = [None, None]   # the step that last read the buffer has been enqueued and finished
    upload_no = [0]

    def upload():
        i = upload_no[0] % 2
        upload_no[0] += 1
        with torch.cuda.stream(copy_stream):
            if free_ev[i] is not None:
                copy_stream.wait_event(free_ev[i])
            dev_bufs[i].copy_(staging, non_blocking=True)
            t = dict(resident)
            for k in io_keys:
                t[k] = view_of(dev_bufs[i], k)
            if host_rows is not None:
                # the loader built the boundaries on the host: no read-back for the range checks
                fr.provide_boundary_rows(t["boundary"], host_rows)
            done = torch.cuda.Event()
            done.record(copy_stream)
        return t, done, i

    def e2e_loop(steps):
        nxt = upload()
        for i in range(steps):
            t, done, buf = nxt
            main_stream.wait_event(done)
            if i + 1 < steps:
                nxt = upload()
            # no L2 flush here: every step works on a fresh 155 MB upload (larger than the
            # 126 MB L2) and moves about 1.5 GB through the cache
            loss = step(t, buf)
            loss_host.copy_(loss, non_blocking=True)
            free_ev[buf] = torch.cuda.Event()
            free_ev[buf].record(main_stream)

    e2e_loop(max(args.warmup, 2))   # at least one step on each upload buffer (graph capture)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    e2e_loop(args.steps)
    ev1.record()
    barrier()
    e2e_total = ev0.elapsed_time(ev1)
    if world > 1:
        tt = torch.tensor([e2e_total], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_total = float(tt.item())
    e2e_ms = e2e_total / args.steps
    h2d = total
    e2e_value = batch * world / (e2e_ms * 1e-3)

    hbm_gbs, peak_kind = measured_peaks()
    line = {"metric": "utterances/sec", "value": round(value, 1), "unit": "utt/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,
            "dtype": ("f32" if args.input_dtype == "f32" else
                      f"f32 arithmetic on {args.input_dtype} inputs (not the benchmark's configuration)"),
            "data": "synthetic", "config": cfg,
            "joiner_impl": joiner_impl[args.joiner],
            "streams": ("one" if args.no_overlap else
                        "two: the simple loss (forward, hence its backward) on a second stream, "
                        "so that its backward overlaps with the pruned branch's"),
            "graph": (graph_note[0] if args.no_graph else
                      "the step (forward + backward, both streams) is captured once per set of input "
                      "buffers with fast_rnnt_b200.graphs.GraphedStep and replayed; the all-reduce of "
                      "the loss and the uploads are not in the graph"),
            "clocks": clocks.summary(),
            "e2e": {"value": round(e2e_value, 1), "unit": "utt/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": 4, "ms_per_step": round(e2e_ms, 4),
                    "h2d_gbs_per_rank": round(h2d / (e2e_ms * 1e-3) / 1e9, 1),
                    "note": "uploads every input of the step, reads back the loss; the input "
                            "gradients (about as many bytes as the inputs) stay on the device, "
                            "where a training step consumes them.  When ms_per_step here exceeds "
                            "the device-resident one, the step is bound by the upload "
                            "(h2d_gbs_per_rank against the host link's rate)"},
            "gpu_launches": int(launches),
            "loss_allreduced": float(last_loss[0]) if last_loss[0] is not None else None}
    if args.workload == "c5" and args.batch is None and C5_GLOBAL_LOSS is not None:
        rel = abs(line["loss_allreduced"] - C5_GLOBAL_LOSS) / abs(C5_GLOBAL_LOSS)
        line["loss_check"] = {"expected": C5_GLOBAL_LOSS, "rel_err": rel,
                              "what": "sum over the global batch of 512 utterances; the same "
                                      "number at every count of ranks"}
        assert rel < 1e-5, line["loss_check"]

    if args.input_dtype != "f32":
        args.no_stages = args.no_cpu_baseline = True
    if rank == 0 and not args.no_stages:
        stages, cells = stage_table(fr, wl, dev, flush, hbm_gbs)
        in_step = STEP_STAGES[args.joiner]
        products = PRODUCT_STAGES[args.joiner]
        step_sum = sum(stages[k]["ms"] for k in in_step)
        prod_sum = sum(stages[k]["ms"] for k in products)
        line["stages"] = stages
        line["step_stages"] = {"launched_by_the_timed_step": in_step,
                               "sum_ms": round(step_sum, 4),
                               "note": "each stage timed alone with a flushed L2; their sum is not "
                                       "the step time (ms_per_step is: stages overlap there), it "
                                       "shows where the time goes"}
        line["loss_path"] = {"ms_per_step": round(step_sum - prod_sum, 4),
                             "value": round(batch / ((step_sum - prod_sum) * 1e-3), 1), "unit": "utt/s",
                             "note": "the stages the timed step launches minus the joiner's three "
                                     "tensor-core products " + str(products) + " (the caller's network)"}
        mi_ms = stages["mi_forward"]["ms"] + stages["mi_backward"]["ms"]
        line["mi_cells_per_s"] = round(cells / (mi_ms * 1e-3), 1)
        line["mi_c2"] = mi_c2_table(dev, flush)
        # the dominant kernel of a step: the slowest of the joiner's products
        tf_peak, tf_kind = measured_tensor_peak()
        if products:
            top = max(products, key=lambda k: stages[k]["ms"])
            pairs = args.joiner == "fused"
            line["roofline"] = {
                "kernel": top + (" (pair_umma_kernel / pair_umma256_kernel, fp16-pair tcgen05)" if pairs else
                                 " (linear_umma_kernel, 3xTF32 tcgen05)"),
                "bound": "tensor", "achieved": stages[top]["tflops"], "peak": tf_peak, "unit": "TFLOP/s",
                "frac": round(stages[top]["tflops"] / tf_peak, 4),
                "peak_kind": f"dense bf16 burst, of {tf_kind}",
                "note": ("achieved counts the useful 2*M*N*K flops of an fp32-accurate product; the "
                         "kernel issues 3x that as fp16 MMAs (hi*hi + hi*lo + lo*hi), so 1/3 of the "
                         "16-bit peak is the ceiling of this formulation" if pairs else
                         "achieved counts the useful 2*M*N*K flops of an fp32-accurate product; the "
                         "kernel issues 3x that as tf32 MMAs, and tf32 runs at half the bf16 rate, so "
                         "1/6 of the bf16 peak is the ceiling of this formulation"),
                "issued_tflops": round(3 * stages[top]["tflops"], 1),
                "traffic": NCU_TRAFFIC_C3.get(top) if args.workload == "c3" else None}
        # and the slowest single-kernel stage among the others the step launches
        single = [k for k in in_step if not k.startswith(("simple_", "fused_")) and k not in products]
        lp = max(single, key=lambda k: stages[k]["ms"])
        line["roofline_loss_path"] = {
            "kernel": lp, "bound": "hbm", "achieved": stages[lp]["gbs"], "peak": hbm_gbs, "unit": "GB/s",
            "frac": stages[lp]["hbm_frac"], "peak_kind": f"of {peak_kind}",
            "traffic": NCU_TRAFFIC_C3.get(lp) if args.workload == "c3" else None,
            "note": ("the mutual-information sweeps are bound by their (S_b+T_b+1)-step dependency "
                     "chain, not by bytes: the fraction is low by construction"
                     if lp.startswith("mi_") else "")}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        sample = min(batch, 16)
        cpu_steps = 20 if args.workload == "c3" else 3   # about 10 s of host work
        v, ms, kind, cpu_loss, cpu_grads = cpu_reference_run(args.workload, sample, cpu_steps, 1)
        what = ("the reference's own python package on its CPU extension" if kind == "reference"
                else "CPU oracle port: torch CPU ops + C recursion")
        line["cpu_baseline"] = {"value": round(v, 3), "unit": "utt/s",
                                "cores": torch.get_num_threads(), "kind": kind,
                                "sample": f"{sample} utterances of the {args.workload} batch, {cpu_steps} "
                                          f"steps ({what})",
                                "ms_per_step": round(ms, 2)}
        # the same utterances through the timed GPU path: loss against the CPU leg's loss
        wl_s = workloads.pipeline_workload(args.workload, batch=sample)
        ts = {k: wl_s[k].to(dev) for k in TENSOR_KEYS}
        gpu_loss = float(make_step(fr, wl_s, args.joiner)(ts))
        line["parity"] = {"cpu_loss": cpu_loss, "gpu_loss": gpu_loss,
                          "rel_err": abs(gpu_loss - cpu_loss) / abs(cpu_loss),
                          "what": f"simple + pruned loss of the CPU leg's {sample} utterances, this "
                                  "library on the GPU (own prune ranges) against the CPU leg"}
        if args.workload == "c3":
            try:
                ref_cuda, noise = reference_cuda_run(args.workload, batch, sample,
                                                     cpu_grads if kind == "reference" else None, dev)
            except Exception as e:  # pragma: no cover
                ref_cuda, noise = {"unavailable": f"{type(e).__name__}: {e}"[:200]}, None
            if ref_cuda is not None:
                line["reference_cuda"] = ref_cuda
            if noise is not None:
                line["noise_floor"] = noise
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
