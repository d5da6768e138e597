"""Writes the golden vectors under tests/golden/ by running the REFERENCE itself.

Usage (only where a checkout of k2-fsa/fast_rnnt and its compiled CPU extension
exist; the committed .npz files are what the tests read):

    make -C oracle ref REF=/path/to/fast_rnnt      # builds oracle/_ref/_fast_rnnt.so
    python tests/golden/make_golden.py --ref /path/to/fast_rnnt

Every array in the .npz files is an output of the reference's own python
package (fast_rnnt/python/fast_rnnt) running on its own CPU extension; inputs
are stored next to the outputs for the small cases, and re-created from the
recorded seed for the full-size configurations (only summaries are stored for
those: per-utterance scores, losses, strided samples of the gradients and the
prune-range starts).
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from tests import workloads  # noqa: E402  (seeded input builders shared with the tests)


def load_reference(ref_root):
    sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
    sys.path.insert(0, os.path.join(ref_root, "fast_rnnt", "python"))
    import _fast_rnnt  # noqa: F401  (must be importable before the package)
    import fast_rnnt
    return fast_rnnt


def npy(x):
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy()
    return np.asarray(x)


def save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **{k: npy(v) for k, v in arrays.items()})
    print(f"{name}.npz  {os.path.getsize(path) / 1024:.1f} KiB")


def sample(x, n=4096):
    """Deterministic strided sample of a tensor (flattened)."""
    flat = x.detach().reshape(-1)
    step = max(1, flat.numel() // n)
    return flat[::step].clone()


def case_basic(fr):
    # the fixed tensors of the reference's own test_rnnt_loss_basic
    # (fast_rnnt/python/tests/rnnt_loss_test.py:70-82) and :391-404
    lm, am, symbols, blank = workloads.reference_basic_tensors()
    px, py = fr.get_rnnt_logprobs(lm=lm, am=am, symbols=symbols, termination_symbol=blank)
    m = fr.mutual_information_recursion(px=px, py=py, boundary=None)
    simple = fr.rnnt_loss_simple(lm=lm, am=am, symbols=symbols, termination_symbol=blank,
                                 boundary=None, reduction="none")
    smoothed0 = fr.rnnt_loss_smoothed(lm=lm, am=am, symbols=symbols, termination_symbol=blank,
                                      lm_only_scale=0.0, am_only_scale=0.0, boundary=None,
                                      reduction="none")
    smoothed = fr.rnnt_loss_smoothed(lm=lm, am=am, symbols=symbols, termination_symbol=blank,
                                     lm_only_scale=0.0, am_only_scale=0.333, boundary=None,
                                     reduction="none")
    logits = am.unsqueeze(2) + lm.unsqueeze(1)
    joint = fr.rnnt_loss(logits=logits, symbols=symbols, termination_symbol=blank,
                         boundary=None, reduction="none")
    out = dict(lm=lm, am=am, symbols=symbols, blank=blank, px=px, py=py, neg_m=-m,
               simple=simple, smoothed0=smoothed0, smoothed_am0333=smoothed, joint=joint)
    try:
        import torchaudio.functional as taf
        out["torchaudio"] = taf.rnnt_loss(
            logits=logits, targets=symbols.int(),
            logit_lengths=torch.tensor([4], dtype=torch.int32),
            target_lengths=torch.tensor([3], dtype=torch.int32),
            blank=blank, reduction="none")
    except Exception as e:  # pragma: no cover
        print("torchaudio unavailable:", e)
    save("basic", **out)


def case_mi(fr):
    # small standalone recursions: dtypes x recursion types x boundary kinds
    for name, kw in workloads.MI_SMALL_CASES.items():
        px, py, boundary = workloads.mi_small(**kw)
        px.requires_grad_(True)
        py.requires_grad_(True)
        scores, (gx, gy) = fr.mutual_information_recursion(px, py, boundary, return_grad=True)
        occ_x, occ_y = gx.clone(), gy.clone()
        w = torch.linspace(0.5, 2.0, px.shape[0], dtype=px.dtype)
        (scores * w).sum().backward()
        joint = fr.joint_mutual_information_recursion(
            (px.detach() * 0.25, px.detach() * 0.75), (py.detach() * 0.25, py.detach() * 0.75),
            boundary)
        save("mi_" + name, px=px, py=py,
             boundary=(boundary if boundary is not None else np.zeros((0, 4), np.int64)),
             scores=scores, occ_x=occ_x, occ_y=occ_y, w=w, px_grad=px.grad, py_grad=py.grad,
             joint=joint)


def run_pipeline(fr, wl, rnnt_type, full_arrays, keep_full=()):
    """The documented usage (reference README.md:150-190): smoothed simple loss
    with return_grad -> ranges -> pruning -> joiner -> pruned loss -> backward.
    Without full_arrays only summaries are kept, plus the arrays named in keep_full."""
    am = wl["am"].clone().requires_grad_(True)
    lm = wl["lm"].clone().requires_grad_(True)
    enc = wl["enc"].clone().requires_grad_(True)
    dec = wl["dec"].clone().requires_grad_(True)
    W = wl["joiner_w"].clone().requires_grad_(True)
    bias = wl["joiner_b"].clone().requires_grad_(True)
    symbols, boundary, blank = wl["symbols"], wl["boundary"], wl["blank"]
    px, py = fr.get_rnnt_logprobs_smoothed(
        lm=lm.detach(), am=am.detach(), symbols=symbols, termination_symbol=blank,
        lm_only_scale=wl["lm_only_scale"], am_only_scale=wl["am_only_scale"],
        boundary=boundary, rnnt_type=rnnt_type)
    simple, (occ_x, occ_y) = fr.rnnt_loss_smoothed(
        lm=lm, am=am, symbols=symbols, termination_symbol=blank,
        lm_only_scale=wl["lm_only_scale"], am_only_scale=wl["am_only_scale"],
        boundary=boundary, rnnt_type=rnnt_type, reduction="sum", return_grad=True)
    occ_x_keep, occ_y_keep = occ_x.clone(), occ_y.clone()
    ranges = fr.get_rnnt_prune_ranges(px_grad=occ_x, py_grad=occ_y, boundary=boundary,
                                      s_range=wl["s_range"])
    am_p, lm_p = fr.do_rnnt_pruning(am=enc, lm=dec, ranges=ranges)
    logits = torch.nn.functional.linear(torch.tanh(am_p + lm_p), W, bias)
    logits.retain_grad()
    ppx, ppy = fr.get_rnnt_logprobs_pruned(
        logits=logits.detach(), symbols=symbols, ranges=ranges, termination_symbol=blank,
        boundary=boundary, rnnt_type=rnnt_type)
    pruned = fr.rnnt_loss_pruned(logits=logits, symbols=symbols, ranges=ranges,
                                 termination_symbol=blank, boundary=boundary,
                                 rnnt_type=rnnt_type, reduction="sum")
    (simple + pruned).backward()
    out = dict(simple=simple, pruned=pruned, s_begin=ranges[:, :, 0].to(torch.int16),
               s_range=ranges.shape[2])
    if not full_arrays:
        out.update(float64_samples(fr, wl, rnnt_type, ranges))
    big = dict(px=px, py=py, occ_x=occ_x_keep, occ_y=occ_y_keep, pruned_px=ppx, pruned_py=ppy,
               am_grad=am.grad, lm_grad=lm.grad, enc_grad=enc.grad, dec_grad=dec.grad,
               logits=logits, logits_grad=logits.grad, w_grad=W.grad, b_grad=bias.grad)
    if full_arrays:
        out.update(big)
        out.update({k: v for k, v in wl.items() if isinstance(v, torch.Tensor)})
    else:
        out.update({k + "_sample": sample(v) for k, v in big.items()})
        out.update({k + "_sum": v.detach().double().clamp(min=-1e30).sum() for k, v in big.items()})
        out.update({k: big[k] for k in keep_full})
    return out


def float64_samples(fr, wl, rnnt_type, ranges):
    """The same pipeline in float64 on the float32 run's ranges: samples of what exact
    arithmetic gives.  |float32 sample - float64 sample| is the reference's own rounding
    noise, the floor below which a comparison with its float32 output means nothing."""
    d = lambda x: x.double().clone().requires_grad_(True)  # noqa: E731
    am, lm, enc, dec, W, bias = (d(wl[k]) for k in ("am", "lm", "enc", "dec", "joiner_w", "joiner_b"))
    symbols, boundary, blank = wl["symbols"], wl["boundary"], wl["blank"]
    simple, (occ_x, occ_y) = fr.rnnt_loss_smoothed(
        lm=lm, am=am, symbols=symbols, termination_symbol=blank,
        lm_only_scale=wl["lm_only_scale"], am_only_scale=wl["am_only_scale"],
        boundary=boundary, rnnt_type=rnnt_type, reduction="sum", return_grad=True)
    occ_x, occ_y = occ_x.clone(), occ_y.clone()
    am_p, lm_p = fr.do_rnnt_pruning(am=enc, lm=dec, ranges=ranges)
    logits = torch.nn.functional.linear(torch.tanh(am_p + lm_p), W, bias)
    logits.retain_grad()
    pruned = fr.rnnt_loss_pruned(logits=logits, symbols=symbols, ranges=ranges,
                                 termination_symbol=blank, boundary=boundary,
                                 rnnt_type=rnnt_type, reduction="sum")
    (simple + pruned).backward()
    big = dict(occ_x=occ_x, occ_y=occ_y, am_grad=am.grad, lm_grad=lm.grad, enc_grad=enc.grad,
               dec_grad=dec.grad, logits=logits, logits_grad=logits.grad, w_grad=W.grad,
               b_grad=bias.grad)
    out = {k + "_f64_sample": sample(v) for k, v in big.items()}
    out.update(simple_f64=simple, pruned_f64=pruned)
    return out


def case_pipelines(fr):
    for rnnt_type in ("regular", "modified", "constrained"):
        wl = workloads.pipeline_workload("mini", rnnt_type=rnnt_type)
        save("pipeline_mini_" + rnnt_type, **run_pipeline(fr, wl, rnnt_type, True))
    # a plain (not smoothed) simple loss and a delay-penalised variant on the mini inputs
    wl = workloads.pipeline_workload("mini", rnnt_type="regular")
    out = {}
    for rnnt_type in ("regular", "modified", "constrained"):
        am = wl["am"].clone().requires_grad_(True)
        lm = wl["lm"].clone().requires_grad_(True)
        loss = fr.rnnt_loss_simple(lm=lm, am=am, symbols=wl["symbols"], termination_symbol=0,
                                   boundary=wl["boundary"], rnnt_type=rnnt_type,
                                   delay_penalty=0.01, reduction="none")
        loss.sum().backward()
        out[f"simple_dp_{rnnt_type}"] = loss
        out[f"simple_dp_{rnnt_type}_am_grad"] = am.grad
        out[f"simple_dp_{rnnt_type}_lm_grad"] = lm.grad
        am = wl["am"].clone().requires_grad_(True)
        lm = wl["lm"].clone().requires_grad_(True)
        loss = fr.rnnt_loss_smoothed(lm=lm, am=am, symbols=wl["symbols"], termination_symbol=0,
                                     lm_only_scale=0.1, am_only_scale=0.2,
                                     boundary=wl["boundary"], rnnt_type=rnnt_type,
                                     reduction="mean")
        loss.backward()
        out[f"smoothed_{rnnt_type}"] = loss
        out[f"smoothed_{rnnt_type}_am_grad"] = am.grad
        out[f"smoothed_{rnnt_type}_lm_grad"] = lm.grad
    save("simple_variants_mini", **out)


def case_c1(fr):
    wl = workloads.config_c1()
    am = wl["am"].clone().requires_grad_(True)
    lm = wl["lm"].clone().requires_grad_(True)
    px, py = fr.get_rnnt_logprobs(lm=lm.detach(), am=am.detach(), symbols=wl["symbols"],
                                  termination_symbol=0, boundary=wl["boundary"])
    loss, (gx, gy) = fr.rnnt_loss_simple(lm=lm, am=am, symbols=wl["symbols"],
                                         termination_symbol=0, boundary=wl["boundary"],
                                         reduction="sum", return_grad=True)
    occ_x, occ_y = gx.clone(), gy.clone()
    loss.backward()
    save("c1_simple", loss=loss, px=px, py=py, occ_x=occ_x, occ_y=occ_y,
         am_grad=am.grad, lm_grad=lm.grad, boundary=wl["boundary"], symbols=wl["symbols"],
         am_sample=sample(wl["am"]), lm_sample=sample(wl["lm"]))


def case_c2(fr):
    out = {}
    for tag, with_boundary in (("full", False), ("bounded", True)):
        px, py, boundary = workloads.config_c2(with_boundary)
        scores, (gx, gy) = fr.mutual_information_recursion(px, py, boundary, return_grad=True)
        out[tag + "_scores"] = scores
        out[tag + "_occ_x_sample"] = sample(gx)
        out[tag + "_occ_y_sample"] = sample(gy)
        out[tag + "_occ_x_sum"] = gx.double().sum()
        out[tag + "_occ_y_sum"] = gy.double().sum()
        out[tag + "_px_sample"] = sample(px)
    save("c2_mi", **out)


def case_c3(fr):
    wl = workloads.pipeline_workload("c3", rnnt_type="regular")
    save("c3_pipeline", **run_pipeline(fr, wl, "regular", False))


def case_c5_shape(fr):
    # the large-vocabulary shape (T=400, S=60, C=5000, s_range=5) on a batch the CPU
    # handles; the occupancies are kept in full so that the range stage can be checked
    # bit for bit on the reference's own inputs
    wl = workloads.pipeline_workload("c5", rnnt_type="regular", batch=3, seed=2)
    save("c5_shape_pipeline", **run_pipeline(fr, wl, "regular", False, keep_full=("occ_x", "occ_y")))


def case_c4(fr):
    wl = workloads.config_c4()
    logits = wl["logits"].clone().requires_grad_(True)
    loss = fr.rnnt_loss(logits=logits, symbols=wl["symbols"], termination_symbol=0,
                        boundary=wl["boundary"], reduction="sum")
    loss.backward()
    out = dict(loss=loss, logits_grad_sample=sample(logits.grad),
               logits_grad_sum=logits.grad.double().sum(), logits_sample=sample(wl["logits"]))
    try:
        import torchaudio.functional as taf
        # torchaudio wants the padded sizes to equal the longest lengths
        t_max = int(wl["boundary"][:, 3].max())
        s_max = int(wl["boundary"][:, 2].max())
        ta = taf.rnnt_loss(logits=wl["logits"][:, :t_max, : s_max + 1].contiguous(),
                           targets=wl["symbols"][:, :s_max].int().contiguous(),
                           logit_lengths=wl["boundary"][:, 3].int(),
                           target_lengths=wl["boundary"][:, 2].int(), blank=0, reduction="sum")
        out["torchaudio_loss"] = ta
    except Exception as e:  # pragma: no cover
        print("torchaudio unavailable:", e)
    save("c4_unpruned", **out)


def case_joint_small(fr):
    for rnnt_type in ("regular", "modified", "constrained"):
        wl = workloads.joint_small(rnnt_type)
        logits = wl["logits"].clone().requires_grad_(True)
        px, py = fr.get_rnnt_logprobs_joint(logits=logits.detach(), symbols=wl["symbols"],
                                            termination_symbol=wl["blank"],
                                            boundary=wl["boundary"], rnnt_type=rnnt_type)
        loss = fr.rnnt_loss(logits=logits, symbols=wl["symbols"], termination_symbol=wl["blank"],
                            boundary=wl["boundary"], rnnt_type=rnnt_type, delay_penalty=0.02,
                            reduction="none")
        loss.sum().backward()
        save("joint_small_" + rnnt_type, logits=wl["logits"], symbols=wl["symbols"],
             boundary=wl["boundary"], blank=wl["blank"], px=px, py=py, loss=loss,
             logits_grad=logits.grad)


def case_prune_edges(fr):
    # s_range larger than S, and tiny T with large S (auto-raised s_range):
    # the two edge cases of rnnt_loss_test.py:520-609 and :615-705
    out = {}
    for tag, wl in workloads.prune_edge_cases().items():
        gx, gy = wl["occ_x"], wl["occ_y"]
        ranges = fr.get_rnnt_prune_ranges(px_grad=gx, py_grad=gy, boundary=wl["boundary"],
                                          s_range=wl["s_range"])
        out[tag + "_occ_x"] = gx
        out[tag + "_occ_y"] = gy
        out[tag + "_boundary"] = wl["boundary"]
        out[tag + "_s_range_in"] = wl["s_range"]
        out[tag + "_ranges"] = ranges
    save("prune_edges", **out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("FAST_RNNT_REFERENCE"), required=False,
                    help="checkout of k2-fsa/fast_rnnt (or set FAST_RNNT_REFERENCE)")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    if not args.ref:
        ap.error("--ref (or FAST_RNNT_REFERENCE) must name a checkout of the reference")
    fr = load_reference(args.ref)
    torch.set_num_threads(max(1, min(8, os.cpu_count() or 1)))
    cases = dict(basic=case_basic, mi=case_mi, pipelines=case_pipelines, c1=case_c1,
                 c2=case_c2, c3=case_c3, c4=case_c4, c5_shape=case_c5_shape, joint_small=case_joint_small,
                 prune_edges=case_prune_edges)
    for name, fn in cases.items():
        if args.only and name not in args.only.split(","):
            continue
        fn(fr)


if __name__ == "__main__":
    main()
