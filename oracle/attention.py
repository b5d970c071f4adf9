"""fp32 attention oracles (CPU, torch). Test infrastructure only.

Shapes used everywhere in this package
  q            [B, Hq, Sq, 128]  bf16
  k, v         [B, Hkv, Skv, 128] bf16
  ids          [B, Hkv, Sq/128, TopK] int32  KV-block ids per query BLOCK,
               shared by the Hq/Hkv query heads of a KV-head group
  counts       [B, Hkv, Sq/128] int32 or None: only ids[..., :count] are live
  O            [B, Hq, Sq, 128] fp32, LSE [B, Hq, Sq] fp32 (natural log)
"""
import math

import torch

BLOCK = 128


def expand_block_ids(ids):
    """[B,Hkv,Sq/128,K] -> per-token lists [B,Hkv,Sq,K], the layout the
    reference masked oracle takes (attention/kv_centric/reference.py:13)."""
    return ids.repeat_interleave(BLOCK, dim=2).contiguous()


@torch.no_grad()
def masked_attention(q, k, v, ids, counts=None, query_chunk=128):
    """The reference's masked-attention computation, generalised.

    Follows attention/kv_centric/reference.py:7-31: build a boolean block
    mask from the selected ids, repeat it to key resolution, fill the
    unselected scores with -inf, softmax, multiply by V, and take logsumexp.
    Generalisations: lists are per query block (not per token), TopK is free,
    and an optional per-row count trims a list (a row with count 0 yields
    O = 0 and LSE = -inf, the neutral element of the log-sum-exp merge).
    """
    bsz, hq, sq, dim = q.shape
    hkv, skv = k.shape[1:3]
    group = hq // hkv
    nblocks = skv // BLOCK
    out = torch.zeros(q.shape, dtype=torch.float32)
    lse = torch.full(q.shape[:-1], -math.inf, dtype=torch.float32)
    for b in range(bsz):
        for h in range(hkv):
            kh, vh = k[b, h].float(), v[b, h].float()
            heads = slice(h * group, (h + 1) * group)
            for first in range(0, sq, query_chunk):
                end = min(first + query_chunk, sq)
                rows = torch.arange(first, end) // BLOCK
                block_mask = torch.zeros((end - first, nblocks), dtype=torch.bool)
                lists = ids[b, h, rows].long()
                if counts is not None:
                    live = torch.arange(ids.shape[-1])[None, :] < counts[b, h, rows].long()[:, None]
                else:
                    live = torch.ones_like(lists, dtype=torch.bool)
                # scatter only live entries
                r_idx = torch.arange(end - first)[:, None].expand_as(lists)
                block_mask[r_idx[live], lists[live]] = True
                mask = block_mask.repeat_interleave(BLOCK, dim=-1)
                scores = (q[b, heads, first:end].float() @ kh.T) / math.sqrt(dim)
                scores = scores.masked_fill(~mask.unsqueeze(0), -math.inf)
                row_lse = torch.logsumexp(scores, dim=-1)
                prob = torch.softmax(scores, dim=-1)
                prob = torch.nan_to_num(prob, nan=0.0)       # fully masked rows
                out[b, heads, first:end] = prob @ vh
                lse[b, heads, first:end] = row_lse
    return out, lse


@torch.no_grad()
def gather_attention(q, k, v, ids, counts=None, q_blocks=None):
    """Same result through the gather formulation.

    Follows attention/q_centric/progression_validation.py:44-62: for each
    (batch, KV head, query block) gather the selected key/value rows and run a
    dense fp32 softmax over them. Adds LSE and the optional counts. `q_blocks`
    restricts the computation to some query blocks (the CPU-baseline slice);
    other rows are left zero / -inf.
    """
    b, hq, sq, dim = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    out = torch.zeros(q.shape, dtype=torch.float32)
    lse = torch.full(q.shape[:-1], -math.inf, dtype=torch.float32)
    offsets = torch.arange(BLOCK)
    todo = range(sq // BLOCK) if q_blocks is None else q_blocks
    for batch in range(b):
        for head in range(hkv):
            for qt in todo:
                n = ids.shape[-1] if counts is None else int(counts[batch, head, qt])
                if n == 0:
                    continue
                pos = (ids[batch, head, qt, :n].long()[:, None] * BLOCK + offsets).flatten()
                queries = q[batch, head * group:(head + 1) * group, qt * BLOCK:(qt + 1) * BLOCK].float()
                keys = k[batch, head].index_select(0, pos).float()
                values = v[batch, head].index_select(0, pos).float()
                s = queries @ keys.T / math.sqrt(dim)
                out[batch, head * group:(head + 1) * group, qt * BLOCK:(qt + 1) * BLOCK] = \
                    torch.softmax(s, dim=-1) @ values
                lse[batch, head * group:(head + 1) * group, qt * BLOCK:(qt + 1) * BLOCK] = \
                    torch.logsumexp(s, dim=-1)
    return out, lse


@torch.no_grad()
def combine_partials(partial_o, partial_lse):
    """Log-sum-exp merge of normalised partial outputs.

    Follows attention/kv_centric/reference.py:34-39 (float64 accumulation):
    L = logsumexp_r L_r, O = sum_r exp(L_r - L) O_r. Shapes [..., R, D] and
    [..., R]. A partial with L_r = -inf has weight 0; if every partial of a row
    is -inf the row is O = 0, L = -inf.
    """
    pl = partial_lse.double()
    lse = torch.logsumexp(pl, dim=-1)
    w = torch.exp(pl - lse.unsqueeze(-1))
    w = torch.nan_to_num(w, nan=0.0)
    po = torch.nan_to_num(partial_o.double(), nan=0.0, posinf=0.0, neginf=0.0) \
        if not torch.isfinite(partial_o).all() else partial_o.double()
    out = (po * w.unsqueeze(-1)).sum(dim=-2)
    return out.float(), lse.float()


def filter_ids_to_range(ids, lo, hi, counts=None):
    """Keep, in order, the ids of every list that fall in [lo, hi): the list a
    KV-split rank owning blocks [lo, hi) sees. Returns (ids', counts') with the
    kept ids packed to the front and the tail filled with `lo`."""
    k = ids.shape[-1]
    live = (ids >= lo) & (ids < hi)
    if counts is not None:
        live &= torch.arange(k)[None, None, None, :] < counts[..., None]
    order = torch.argsort((~live).to(torch.int8), dim=-1, stable=True)
    packed = torch.gather(ids, -1, order)
    cnt = live.sum(-1).to(torch.int32)
    packed = torch.where(torch.arange(k)[None, None, None, :] < cnt[..., None], packed,
                         torch.full_like(packed, lo))
    return packed.contiguous(), cnt.contiguous()
