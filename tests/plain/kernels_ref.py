"""Plain PyTorch restatements of each kernel's contract, one function per kernel, fp32/fp64 on any
device.  Used by the per-kernel GPU tests at sizes other than the engine's."""
import math

import torch


def embedding_ref(ids, table):
    return table.float()[ids.long()]


def rmsnorm_ref(x, w, eps, rows=None):
    x = x.double()
    if rows is not None:
        x = x[rows.long()]
    return (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()).float()


def rope_kv_write_ref(qkv, positions, slot_mapping, kv_cache, nh, nkv, hd, page_size, theta, rotary=True):
    """Returns q [T, nh*hd] (fp32) and writes k, v (fp32 values) into a float copy of kv_cache, returned."""
    T = qkv.shape[0]
    x = qkv.double().view(T, nh + 2 * nkv, hd)
    half = hd // 2
    d = torch.arange(half, dtype=torch.float64, device=qkv.device)
    freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2.0 * d / hd)
    ang = positions.double()[:, None] * freq[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    rot = x[:, :nh + nkv]
    if rotary:
        x0, x1 = rot[..., :half], rot[..., half:]
        rot = torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)
    q = rot[:, :nh].reshape(T, nh * hd).float()
    k, v = rot[:, nh:], x[:, nh + nkv:]
    cache = None
    if kv_cache is not None:
        cache = kv_cache.float().clone()
        for t in range(T):
            s = int(slot_mapping[t])
            if s < 0:
                continue
            page, off = s // page_size, s % page_size
            cache[page, 0, :, off, :] = k[t].float()
            cache[page, 1, :, off, :] = v[t].float()
    return q, cache


def silu_mul_interleaved_ref(gu):
    g, u = gu.double()[:, 0::2], gu.double()[:, 1::2]
    return (g / (1.0 + torch.exp(-g)) * u).float()


def gemm_ref(a, w, bias=None):
    y = a.double() @ w.double().t()
    if bias is not None:
        y = y + bias.double()
    return y.float()


def paged_attention_ref(q, kv_cache, block_table, tok_req, positions, nh, nkv, hd, page_size, window=0, scale=None):
    """Every token attends to positions max(0,p-window+1)..p of its request, gathered through the table."""
    T = q.shape[0]
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    out = torch.zeros(T, nh, hd, dtype=torch.float64, device=q.device)
    qd = q.double().view(T, nh, hd)
    cache = kv_cache.double()
    group = nh // nkv
    for t in range(T):
        p = int(positions[t])
        lo = max(0, p - window + 1) if window and window > 0 else 0
        table = block_table[int(tok_req[t])]
        idx = torch.arange(lo, p + 1, device=q.device)
        pages = table[(idx // page_size).long()].long()
        offs = (idx % page_size).long()
        k = cache[pages, 0, :, offs, :]          # [n, nkv, hd]
        v = cache[pages, 1, :, offs, :]
        for h in range(nh):
            s = (k[:, h // group, :] @ qd[t, h]) * scale
            pr = torch.softmax(s, dim=0)
            out[t, h] = pr @ v[:, h // group, :]
    return out.view(T, nh * hd).float()


def argmax_ref(logits):
    return torch.argmax(logits, dim=-1).to(torch.int32)


def sample_probabilities_ref(row, temperature, top_k, top_p):
    """The reference's pipeline (src/inference/sampler.cpp:197-316) in float64; returns kept probabilities."""
    p = torch.softmax(row.double() / temperature, dim=0)
    if 0 < top_k < p.numel():                       # k at least the vocabulary: nothing is cut
        kth = torch.topk(p, top_k).values[-1]
        p = torch.where(p >= kth, p, torch.zeros_like(p))
        p = p / p.sum()
    if top_p < 1.0:
        sp, _ = torch.sort(p, descending=True)
        c = torch.cumsum(sp, 0)
        cutoff = int((c > top_p).nonzero()[0]) + 1 if bool((c > top_p).any()) else p.numel()
        thr = sp[cutoff - 1]
        p = torch.where(p >= thr, p, torch.zeros_like(p))
        p = p / p.sum()
    return p
