"""Kernel micro-benchmarks (CUDA-event timed, L2 flushed between iterations) and small cases for profilers.

    python -m uttt_b200.ops.microbench [--kernel NAME] [--small] [--iters N]

Kernels: gg_nt, gg_swiglu, gg_write, gg_nn, gg_tn, bmm_nt, dense, swa_fwd, swa_bwd, rms_norm, add_rms_norm, embedding, rope, fw_qk_prep, router, pool_step, plucker,
swiglu, permute, patch_decode, frob, fw_write_pw, adamw, ce.  ``--small`` runs one small case
of the chosen kernel (inputs above L2 size, a few hundred MB on the device) three times, which is what the
profile summaries under ``profiles/`` were captured from.  Prints one JSON line per case with the achieved
TFLOP/s or GB/s and the fraction of the measured peaks in ``MEASURED_PEAKS.json`` when present, and a last line
with the SM clock (median, maximum) and the throttle reasons sampled while the cases ran.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from ..utils.clocks import ClockSampler
from . import functional as F
from ._ext import load


def _peaks():
    for cand in ("MEASURED_PEAKS.json", os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")):
        try:
            with open(cand) as fh:
                d = json.load(fh)
                return d["hbm_gbs"], d["bf16_tflops"]
        except Exception:
            continue
    return 6650.0, 1590.0


def _time(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()                      # 256 MB write: evicts the 126 MB L2
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def _plan(bsz, tokens_heads, experts, topk, dev):
    idx = torch.randint(0, experts, (bsz, tokens_heads, topk), device=dev)
    if topk > 1:
        idx[..., 1] = (idx[..., 0] + 1 + torch.randint(0, experts - 1, idx[..., 0].shape, device=dev)) % experts
    return F.build_group_plan(idx, experts)


def run(kernel: str, small: bool, iters: int):
    dev = torch.device("cuda")
    load(required=True)
    hbm, tflops = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bsz = 1 if small else 4
    d, inter, experts = 384, 1536, 32
    plan = _plan(bsz, 2048 * 4, experts, 2, dev)
    rows, g = plan.rows_padded, plan.num_groups
    real = int(plan.sizes.sum())
    out = []

    def rec(name, ms, flops=None, bytes_=None, **extra):
        r = {"kernel": name, "ms": round(ms, 4), **extra}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["frac_of_measured_bf16"] = round(flops / ms / 1e9 / tflops, 3)
        if bytes_:
            r["gbs"] = round(bytes_ / ms / 1e6, 1)
            r["frac_of_measured_hbm"] = round(bytes_ / ms / 1e6 / hbm, 3)
        print(json.dumps(r), flush=True)
        out.append(r)

    bf = dict(device=dev, dtype=torch.bfloat16)
    for pairs in (False, True):
        # the grouped NT / NN products as one-CTA kernels and as CTA pairs (cta_group::2)
        F.set_cta_pairs(pairs)
        tag = " 2cta" if pairs else " 1cta"
        if kernel in ("gg_nt", "all"):
            x = torch.randn(rows, d, **bf)
            w = torch.randn(g, 2 * inter, d, **bf) * 0.05
            ms = _time(lambda: F.gg_nt(x, w, plan), iters, flush)
            rec("gg_nt[read gate|up]" + tag, ms, flops=2.0 * real * d * 2 * inter, rows=rows, real_rows=real, K=d,
                N=2 * inter)
            h = torch.randn(rows, inter, **bf)
            w1 = torch.randn(g, d, inter, **bf) * 0.05
            ms = _time(lambda: F.gg_nt(h, w1, plan), iters, flush)
            rec("gg_nt[read down]" + tag, ms, flops=2.0 * real * d * inter, rows=rows, real_rows=real, K=inter, N=d)
        if kernel in ("gg_swiglu", "all"):
            x = torch.randn(rows, d, **bf)
            w = torch.randn(g, 2 * inter, d, **bf) * 0.05
            ms = _time(lambda: F.gg_swiglu(x, w, plan), iters, flush)
            rec("gg_swiglu[read gate|up + SwiGLU epilogue]" + tag, ms, flops=2.0 * real * d * 2 * inter, rows=rows,
                real_rows=real, K=d, N=2 * inter)
            if not pairs:
                ms = _time(lambda: F.swiglu(F.gg_nt(x, w, plan)), iters, flush)
                rec("gg_nt + swiglu_fwd [unfused pair of kernels]", ms, flops=2.0 * real * d * 2 * inter)
        if kernel in ("gg_write", "all"):
            ext = load()
            x = torch.randn(rows, d, **bf)
            w = torch.randn(g, 2 * inter, d, **bf) * 0.05
            dh = torch.randn(rows, inter, **bf)
            lr = torch.rand(rows, 3, device=dev)
            ms = _time(lambda: F._swiglu_bwd_kernel(x, w, dh, lr, plan, True, False), iters, flush)
            rec("gg_nt_swiglu_bwd[write: dy02*lr, h*lr1]" + tag, ms, flops=2.0 * real * d * 2 * inter, rows=rows,
                real_rows=real)
            ms = _time(lambda: F._swiglu_bwd_kernel(x, w, dh, None, plan, False, False), iters, flush)
            rec("gg_nt_swiglu_bwd[read backward: dy02]" + tag, ms, flops=2.0 * real * d * 2 * inter)
            if not pairs:
                ms = _time(lambda: ext.fw_write_pw_fwd(F.gg_nt(x, w, plan), dh, lr), iters, flush)
                rec("gg_nt + fw_write_pw_fwd [unfused pair of kernels]", ms, flops=2.0 * real * d * 2 * inter)
        if kernel in ("gg_nn", "all"):
            v = torch.randn(rows, d, **bf)
            w1 = torch.randn(g, d, inter, **bf) * 0.05
            ms = _time(lambda: F.gg_nn(v, w1, plan), iters, flush)
            rec("gg_nn[write dh]" + tag, ms, flops=2.0 * real * d * inter, K=d, N=inter)
            a2 = torch.randn(rows, 2 * inter, **bf)
            w02 = torch.randn(g, 2 * inter, d, **bf) * 0.05
            ms = _time(lambda: F.gg_nn(a2, w02, plan), iters, flush)
            rec("gg_nn[d rows: K 3072, N 384]" + tag, ms, flops=2.0 * real * d * 2 * inter, K=2 * inter, N=d)
    F.set_cta_pairs(True)
    if kernel in ("gg_tn", "all"):
        a = torch.randn(rows, 2 * inter, **bf)
        b = torch.randn(rows, d, **bf)
        ms = _time(lambda: F.gg_tn(a, b, plan), iters, flush)
        rec("gg_tn[G02]", ms, flops=2.0 * real * d * 2 * inter, M=2 * inter, N=d, groups=g)
    if kernel in ("bmm_nt", "all"):
        n = g * 2
        x = torch.randn(n, d, inter, **bf)
        ms = _time(lambda: F.bmm_nt(x, x), iters, flush)
        rec("bmm_nt[NS X X^T]", ms, flops=2.0 * n * d * d * inter, batch=n)
    if kernel in ("dense", "all"):
        # the dense projections of a block (tokens x d -> mlp, mlp -> d, d -> d) on the own batched kernel and on cuBLAS
        for (m_, k_, n_) in ((8192, 1536, 4096), (8192, 4096, 1536), (8192, 1536, 1536), (8192, 1536, 8192)):
            x = torch.randn(1, m_, k_, **bf)
            w = torch.randn(1, n_, k_, **bf) * 0.05
            ms = _time(lambda: F.bmm_nt(x, w), iters, flush)
            rec(f"dense NT own [{m_}x{k_} @ {n_}x{k_}^T]", ms, flops=2.0 * m_ * k_ * n_)
            ms_lib = _time(lambda: torch.mm(x[0], w[0].t()), iters, flush)
            rec(f"dense NT cuBLAS [{m_}x{k_} @ {n_}x{k_}^T]", ms_lib, flops=2.0 * m_ * k_ * n_,
                own_over_library=round(ms_lib / ms, 3))
    if kernel in ("swa_fwd", "all"):
        b_, lq, lk, h, hd, win = bsz, 2048, 4096, 16, 96, 2048
        q = torch.randn(b_, lq, h, hd, **bf)
        k = torch.randn(b_, lk, h, hd, **bf)
        v = torch.randn(b_, lk, h, hd, **bf)
        ms = _time(lambda: F.swa_attention(q, k, v, win, True), iters, flush)
        band = win + 64          # average visible keys per query, rounded up to the tile edge
        rec("swa_fwd[hd96 w2048]", ms, flops=4.0 * b_ * h * lq * band * hd, lq=lq, lk=lk)
    if kernel in ("swa_bwd", "all"):
        ext = load()
        b_, lq, lk, h, hd, win = bsz, 2048, 4096, 16, 96, 2048
        q = torch.randn(b_, lq, h, hd, **bf)
        k = torch.randn(b_, lk, h, hd, **bf)
        v = torch.randn(b_, lk, h, hd, **bf)
        o, lse = ext.swa_fwd(q, k, v, win, True, hd ** -0.5)
        do = torch.randn_like(o)
        ms = _time(lambda: ext.swa_bwd(do, q, k, v, o, lse, win, True, hd ** -0.5), iters, flush)
        band = win + 64
        # five products in the textbook backward (the two-kernel split recomputes S and dP once more)
        rec("swa_bwd[hd96 w2048]", ms, flops=10.0 * b_ * h * lq * band * hd, lq=lq, lk=lk)
    if kernel in ("rms_norm", "all"):
        x = torch.randn(bsz * 2048 * 8, 1536, **bf)
        w = torch.ones(1536, **bf)
        ms = _time(lambda: F.rms_norm(x, w, 1e-6), iters, flush)
        rec("rms_norm_fwd", ms, bytes_=2.0 * x.numel() * 2)
    if kernel in ("add_rms_norm", "all"):
        x = torch.randn(bsz * 2048 * 8, 1536, **bf)
        dl = torch.randn_like(x)
        w = torch.ones(1536, **bf)
        ms = _time(lambda: F.add_rms_norm(x, dl, w, 1e-6), iters, flush)
        rec("add_rms_norm_fwd", ms, bytes_=4.0 * x.numel() * 2)          # two reads, two writes
    if kernel in ("embedding", "all"):
        table = torch.randn(32000, 1536, **bf)
        ids = (torch.rand(bsz, 32768 if not small else 8192, device=dev) ** 3 * 32000).long().clamp_(0, 31999)
        ms = _time(lambda: F.embedding(ids, table), iters, flush)
        rec("embedding_fwd", ms, bytes_=2.0 * ids.numel() * 1536 * 2)
        gy = torch.randn(*ids.shape, 1536, **bf)
        ext = load()
        ms = _time(lambda: ext.embedding_bwd(gy, ids, 32000), iters, flush)
        # read dy once, zero and reduce into the fp32 table
        rec("embedding_bwd[fp32 reductions]", ms, bytes_=ids.numel() * 1536 * 2.0 + 2.0 * 32000 * 1536 * 4)
    if kernel in ("rope", "all"):
        q = torch.randn(bsz, 2048, 16, 96, **bf)
        ms = _time(lambda: F.rope(q, 0, 10000.0), iters, flush)
        rec("rope[hd96]", ms, bytes_=2.0 * q.numel() * 2)
    if kernel in ("fw_qk_prep", "all"):
        x = torch.randn(bsz, 2048, 1536, **bf)
        sc = torch.ones(1536, **bf)
        sh = torch.zeros(1536, **bf)
        ms = _time(lambda: F.fw_qk_prep(x, sc, sh, 4, 96, 10000.0, 0, True, "l2"), iters, flush)
        rec("fw_qk_prep_fwd", ms, bytes_=2.0 * x.numel() * 2)
    if kernel in ("router", "all"):
        rows_r = torch.randn(bsz, 8192, d, **bf)
        rt = torch.randn(experts, d, device=dev) * 0.1
        ms = _time(lambda: F.route_softmax_topk(rows_r, rt, None, 2), iters, flush)
        rec("router_fwd[E32 top2]", ms, bytes_=rows_r.numel() * 2.0 + bsz * 8192 * (experts * 4 + 16),
            flops=2.0 * bsz * 8192 * d * experts)
    if kernel in ("pool_step", "all"):
        m = torch.randn(bsz, experts, 2 * inter, d, device=dev)
        dd = torch.randn(bsz, experts, 2 * inter, d, **bf)
        ms = _time(lambda: F.pool_step(m, dd, 0.1, "restore"), iters, flush)
        rec("pool_step_fwd[restore]", ms, bytes_=float(m.numel()) * (4 + 2 + 4 + 2))
    if kernel in ("plucker", "all"):
        v_, hw = 6, 256
        img = torch.rand(bsz, v_, 3, hw, hw, device=dev)
        fx = torch.tensor([300.0, 300.0, 128.0, 128.0], device=dev).expand(bsz, v_, 4).contiguous()
        c2w = torch.eye(4, device=dev).expand(bsz, v_, 4, 4).contiguous()
        tgt = torch.zeros(v_, dtype=torch.bool, device=dev)
        ms = _time(lambda: F.plucker_embed(img, fx, c2w, tgt, 8), iters, flush)
        rec("plucker_embed[256px]", ms, bytes_=float(img.numel()) * 4 + bsz * v_ * hw * hw * 12 * 4.0)
    if kernel in ("swiglu", "all"):
        y02 = torch.randn(rows, 2 * inter, **bf)
        ms = _time(lambda: F.swiglu(y02), iters, flush)
        rec("swiglu_fwd", ms, bytes_=2.0 * rows * inter * 3)
    if kernel in ("permute", "all"):
        xr = torch.randn(bsz * 8192, d, **bf)
        ms = _time(lambda: F.permute_rows(xr, plan), iters, flush)
        rec("permute_rows[top2]", ms, bytes_=2.0 * xr.numel() * 3)
        yp = torch.randn(rows, d, **bf)
        wts = torch.rand(bsz * 8192, 2, device=dev)
        ms = _time(lambda: F.unpermute_rows(yp, plan, wts), iters, flush)
        rec("unpermute_rows[top2]", ms, bytes_=2.0 * xr.numel() * 3)
    if kernel in ("patch_decode", "all"):
        v_, hw = 4, 256
        yl = torch.randn(bsz, v_ * (hw // 8) ** 2, 192, **bf)
        tg = torch.rand(bsz, v_, 3, hw, hw, device=dev)
        ms = _time(lambda: F.patch_decode(yl, tg, v_, hw, hw, 8), iters, flush)
        rec("patch_decode_fwd[256px]", ms, bytes_=float(yl.numel()) * 2 + tg.numel() * 8.0)
    if kernel in ("frob", "all"):
        gmat = torch.randn(bsz * experts * 2, inter, d, device=dev)
        ms = _time(lambda: F._FrobNormalize.apply(gmat, 1e-7), iters, flush)
        rec("frob_normalize_fwd", ms, bytes_=float(gmat.numel()) * (4 + 4 + 2))
    if kernel in ("fw_write_pw", "all"):
        ext = load()
        y02 = torch.randn(rows, 2 * inter, **bf)
        dh = torch.randn(rows, inter, **bf)
        lr = torch.rand(rows, 3, device=dev)
        ms = _time(lambda: ext.fw_write_pw_fwd(y02, dh, lr), iters, flush)
        rec("fw_write_pw_fwd", ms, bytes_=2.0 * rows * inter * 6)
    if kernel in ("adamw", "all"):
        ext = load()
        n = (32 if small else 256) << 20
        p = torch.randn(n, device=dev)
        gr = torch.randn(n, **bf)
        m, v2 = torch.zeros_like(p), torch.zeros_like(p)
        lo = torch.empty(n, **bf)
        one = torch.ones(1, device=dev)
        ms = _time(lambda: ext.adamw_flat(p, gr, m, v2, lo, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, one, one, 1.0, n), iters, flush)
        rec("adamw_flat", ms, bytes_=float(n) * (4 * 3 * 2 + 2 + 2))
    if kernel in ("ce", "all"):
        ext = load()
        t, vsz = (2048 if small else 8192), 32000
        logits = torch.randn(t, vsz, **bf)
        labels = torch.randint(0, vsz, (t,), device=dev)
        loss = torch.zeros(1, device=dev)
        ms = _time(lambda: ext.ce_fwd_bwd_(logits, labels, loss, -100), iters, flush)
        rec("ce_fwd_bwd", ms, bytes_=float(t) * vsz * 2 * 3)
    status = int(load().gemm_status(torch.zeros(1, device=dev))[0])
    assert status == 0, f"kernel wait timed out (code {status})"
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    try:
        run(args.kernel, args.small, 3 if args.small else args.iters)
    finally:
        print(json.dumps({"clocks": sampler.stop()}), flush=True)


if __name__ == "__main__":
    main()
