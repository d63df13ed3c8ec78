"""Backward mode ``cross_layer_cut`` of the shared-pool model.

Forward values are those of mode ``full``.  In backward, the one shared bank is treated as ``L``
per-reader *streams* (aliases with equal values): reader layer ``l`` reads stream ``l``, and the gradient
that arrives on stream ``l`` after a chunk-boundary write reaches only writer ``l``'s raw inner gradient
``G_l`` (and ``1/L`` of it the writer's momentum gate) plus stream ``l``'s previous master / momentum; the
other writers' contributions enter stream ``l`` as constants.

Behavioural reference: uttt_llm/flame/custom_models/uttt_moe/modeling_recurrent_lact.py
``CrossLayerCutAggregateUpdate`` (:1379-1529), ``_forward_cross_layer_cut`` (:2694-2824) and the
chunk-boundary update (:2568-2692).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from . import fast_weights as fw


class _Alias(torch.autograd.Function):
    """``n`` views of one tensor whose gradients stay separate (summed only at the source)."""

    @staticmethod
    def forward(ctx, n, x):
        ctx.n = n
        return tuple(x.view_as(x) for _ in range(n))

    @staticmethod
    def backward(ctx, *grads):
        total = None
        for g in grads:
            if g is not None:
                total = g if total is None else total + g
        return None, total


def alias_streams(state: fw.PoolState, n: int) -> List[fw.PoolState]:
    cols = []
    for t in state.tensors():
        cols.append([None] * n if t is None else list(_Alias.apply(n, t)))
    return [fw.PoolState(*[c[i] for c in cols]) for i in range(n)]


class CrossLayerCutUpdate(torch.autograd.Function):
    """flat inputs: L x (m02, m1, z02, z1) stream states, L x (G02, G1) raw gradients, L momentum gates.
    outputs: L x (w02, w1, m02, m1, z02, z1)."""

    @staticmethod
    def forward(ctx, update_fn, n, vjp_group, *flat):
        states = [flat[4 * i:4 * i + 4] for i in range(n)]
        grads = [flat[4 * n + 2 * i:4 * n + 2 * i + 2] for i in range(n)]
        gates = list(flat[6 * n:7 * n])
        with torch.no_grad():
            a02 = torch.zeros_like(states[0][0])
            a1 = torch.zeros_like(states[0][1])
            for g02, g1 in grads:
                a02 = a02 + g02
                a1 = a1 + g1
            m = torch.stack(gates, 0).mean(0)
            outs = update_fn(a02, a1, *states[0], m)
        ctx.update_fn, ctx.n, ctx.vjp_group = update_fn, n, max(1, int(vjp_group))
        ctx.save_for_backward(a02, a1, *states[0], m)
        ctx.gate_dtypes = [g.dtype for g in gates]
        result = []
        for _ in range(n):
            result.extend(o.view_as(o) for o in outs)
        return tuple(result)

    @staticmethod
    def backward(ctx, *gout):
        n = ctx.n
        a02, a1, m02, m1, z02, z1, m = ctx.saved_tensors
        bsz = a02.shape[0]
        d_state = [(None, None, None, None)] * n
        d_raw = [(None, None)] * n
        d_gate = [None] * n
        for start in range(0, n, ctx.vjp_group):
            streams = [i for i in range(start, min(n, start + ctx.vjp_group))
                       if any(gout[6 * i + j] is not None for j in range(6))]
            if not streams:
                continue
            cnt = len(streams)

            def rep(t):
                return t.detach().repeat(cnt, *([1] * (t.dim() - 1))).requires_grad_(True)

            with torch.enable_grad():
                ins = [rep(t) for t in (a02, a1, m02, m1, z02, z1, m)]
                outs = ctx.update_fn(*ins)
                cots = []
                for j, o in enumerate(outs):
                    parts = [torch.zeros_like(o[:bsz]) if gout[6 * i + j] is None else gout[6 * i + j].to(o.dtype)
                             for i in streams]
                    cots.append(torch.cat(parts, 0))
                g = torch.autograd.grad(outs, ins, cots, allow_unused=True)
            for pos, i in enumerate(streams):
                rows = slice(pos * bsz, (pos + 1) * bsz)
                take = [None if t is None else t[rows] for t in g]
                d_raw[i] = (take[0], take[1])
                d_state[i] = (take[2], take[3], take[4], take[5])
                d_gate[i] = None if take[6] is None else (take[6] / n).to(ctx.gate_dtypes[i])
        flat = []
        for i in range(n):
            flat.extend(d_state[i])
        for i in range(n):
            flat.extend(d_raw[i])
        flat.extend(d_gate)
        return (None, None, None, *flat)


def cross_layer_cut_write(model, states: Sequence[fw.PoolState], feats, offset: int):
    """Chunk-boundary write with per-reader streams.  Returns (new stream states, probs, counts)."""
    cfg = model.config
    n = len(model.layers)
    dt = states[0].w02.dtype

    def _writers(*args):
        outs = []
        for li, layer in enumerate(model.layers):
            x_in, k_flat, v_flat, w02, w1 = args[5 * li:5 * li + 5]
            g02, g1, m, p, c = layer.raw_grad(x_in, k_flat, v_flat, w02, w1, model._router(li),
                                              model._router_bias(li), offset)
            outs.extend([g02, g1, m, p, c])
        return tuple(outs)

    wargs = []
    for li in range(n):
        wargs.extend([*feats[li], states[li].w02, states[li].w1])
    wout = model._ckpt(_writers, *wargs)
    raw = [(wout[5 * i], wout[5 * i + 1]) for i in range(n)]
    gates = [wout[5 * i + 2] for i in range(n)]
    if getattr(model, "ep", None) is not None:
        # expert parallelism: the owner of an expert updates every sequence of the group, so it needs their gates
        gates = [model.ep.gather_sequences(g.reshape(-1)) for g in gates]
    probs = torch.stack([wout[5 * i + 3] for i in range(n)]).float()
    counts = torch.stack([wout[5 * i + 4] for i in range(n)]).float()

    def update_fn(a02, a1, m02, m1, z02, z1, m):
        st = fw.PoolState(None, None, m02, m1, z02, z1)
        new = fw.apply_pool_update(a02, a1, st, m.view(-1, 1, 1, 1), cfg.memory_aggregate_lr_scale, cfg.use_moun,
                                   compute_dtype=dt)
        return new.w02, new.w1, new.m02, new.m1, new.z02, new.z1

    flat = []
    for s in states:
        flat.extend([s.m02, s.m1, s.z02, s.z1])
    for g02, g1 in raw:
        flat.extend([g02, g1])
    flat.extend(gates)
    out = CrossLayerCutUpdate.apply(update_fn, n, cfg.memory_cross_layer_cut_vjp_group, *flat)
    new_states = [fw.PoolState(*out[6 * i:6 * i + 6]) for i in range(n)]
    return new_states, probs, counts
