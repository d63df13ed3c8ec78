"""Cached inference for the chunk-recurrent models (``use_cache=True`` in eval mode) and a small
``generate`` helper.

Cache protocol (the counterpart of uttt_llm/flame/custom_models/lact_cache_utils.py:32-87 and
``_forward_with_generation_cache``, modeling_recurrent_lact.py:3162-3385): tokens of the current chunk
are processed incrementally against (carried window history ++ this chunk's keys so far) and read the
pool state as it was at the chunk start; the per-layer write inputs of the chunk are accumulated, and
the pool update fires when the first token of the *next* chunk arrives.  Fragments are not replayed:
the result equals the one-shot forward up to floating-point rounding of the fragment boundaries.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional

import torch

from .common import trim_history


@dataclass
class GenerationCache:
    states: List[Any]
    hist: List[Any]                       # per layer (k, v) of the previous chunks (window history)
    chunk_kv: List[Any]                   # per layer (k, v) of the current chunk so far
    feats: List[List[Any]]                # per layer list of (x_attn_in, x_memory_in, xi_out, k_flat, v_flat) fragments
    chunk_start: int = 0
    chunk_fill: int = 0
    seen_tokens: int = 0

    def reorder(self, beam_idx: torch.Tensor) -> "GenerationCache":
        def sel(t):
            return None if t is None else t.index_select(0, beam_idx)
        self.states = [type(s)(*[sel(t) for t in s.tensors()]) for s in self.states]
        self.hist = [(sel(k), sel(v)) for k, v in self.hist]
        self.chunk_kv = [(sel(k), sel(v)) for k, v in self.chunk_kv]
        self.feats = [[tuple(sel(t) for t in frag) for frag in layer] for layer in self.feats]
        return self


def _cat(a, b):
    return b if a is None else torch.cat([a, b], dim=1)


@torch.no_grad()
def forward_with_cache(model, inputs_embeds: torch.Tensor, past: Optional[GenerationCache]):
    cfg = model.config
    chunk = cfg.chunk_size
    bsz, total, _ = inputs_embeds.shape
    n_layers = len(model.layers)
    if past is None:
        past = GenerationCache(states=model.init_states(bsz), hist=[(None, None)] * n_layers,
                               chunk_kv=[(None, None)] * n_layers, feats=[[] for _ in range(n_layers)])
    keep = model.layers[0].attn.history_len(chunk) if cfg.window_size is not None else None
    outputs = []
    pos = 0
    shared = not getattr(model, "per_layer_pool", False)
    while pos < total:
        if past.chunk_fill == chunk:
            if cfg.use_memory_block:
                keys = ("x_attn_in", "x_memory_in", "xi_out", "attn_k", "attn_v")
                caches = [{k: torch.cat([f[i] for f in frags], dim=1) for i, k in enumerate(keys)}
                          for frags in past.feats]
                # the same composition of the write's inputs as in training (gapped layers, projections of a feature)
                if hasattr(model, "compose_write_inputs"):
                    feats = model.compose_write_inputs(caches)
                else:
                    feats = [(c["x_attn_in"], c["attn_k"], c["attn_v"]) for c in caches]
                past.states, _, _ = model._chunk_write(past.states, feats, past.chunk_start)
            past.hist = [trim_history(hk, hv, ck, cv, keep) for (hk, hv), (ck, cv) in zip(past.hist, past.chunk_kv)]
            past.chunk_kv = [(None, None)] * n_layers
            past.feats = [[] for _ in range(n_layers)]
            past.chunk_start += chunk
            past.chunk_fill = 0
        take = min(total - pos, chunk - past.chunk_fill)
        h = inputs_embeds[:, pos:pos + take]
        offset = past.chunk_start + past.chunk_fill
        for li, layer in enumerate(model.layers):
            st = past.states[0] if shared else past.states[li]
            hk, hv = past.hist[li]
            ck, cv = past.chunk_kv[li]
            k_ctx = ck if hk is None else (hk if ck is None else torch.cat([hk, ck], dim=1))
            v_ctx = cv if hv is None else (hv if cv is None else torch.cat([hv, cv], dim=1))
            if cfg.use_memory_block:
                out = layer(h, k_ctx, v_ctx, st.w02, st.w1, model._router(li), model._router_bias(li), offset)
            else:
                out = layer(h, k_ctx, v_ctx, None, None, None, None, offset)
            h, x_in, k_flat, v_flat, k_rot, v_new = out[:6]
            past.chunk_kv[li] = (_cat(ck, k_rot), _cat(cv, v_new))
            past.feats[li].append((x_in, out[8] if len(out) > 8 else x_in, h, k_flat, v_flat))
        outputs.append(h)
        pos += take
        past.chunk_fill += take
        past.seen_tokens += take
    hidden = model.norm(torch.cat(outputs, dim=1))
    return hidden, hidden.new_zeros((), dtype=torch.float32), None, past


@torch.no_grad()
def generate(lm, input_ids: torch.Tensor, max_new_tokens: int = 32, temperature: float = 0.0,
             eos_token_id: Optional[int] = None) -> torch.Tensor:
    """Greedy / temperature sampling with the chunk-recurrent cache."""
    lm.eval()
    out = lm(input_ids=input_ids, use_cache=True, logits_to_keep=1)
    cache = out.past_key_values
    tokens = input_ids
    for _ in range(max_new_tokens):
        logits = out.logits[:, -1].float()
        if temperature > 0:
            nxt = torch.multinomial(torch.softmax(logits / temperature, -1), 1)
        else:
            nxt = logits.argmax(-1, keepdim=True)
        tokens = torch.cat([tokens, nxt], dim=1)
        if eos_token_id is not None and bool((nxt == eos_token_id).all()):
            break
        out = lm(input_ids=nxt, past_key_values=cache, use_cache=True, logits_to_keep=1)
        cache = out.past_key_values
    return tokens
