"""Whole-sequence LLaMA decoder written from the reference's formulas.

Every function names the file:line of Cyxuan0311/Forge that it restates.  No
cache, no batching, no fusing: one request, all of its tokens, every time.
Default arithmetic is float64 on the CPU so that the oracle's own rounding is
far below the tolerances of the engine under test.
"""
import json
import math
import os

import torch

from .safetensors_reader import read_safetensors


def embedding(ids, table):
    """h[t,:] = E[id_t,:]   (src/operators/cpu/embedding.cpp:248-260; cuda_embedding.cu:9-25)."""
    return table[ids.long()]


def rms_norm(x, weight, eps):
    """y = x * 1/sqrt(mean(x^2)+eps) * w   (src/operators/cpu/norm.cpp:98-112; cuda_rms_norm.cu:10-36)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(ms + eps)) * weight


def linear(x, weight, bias=None):
    """y = x . W^T (+ b), W is [out,in]   (src/operators/cpu/matmul.cpp:1134-1148, bias :1005-1036)."""
    y = x @ weight.t()
    if bias is not None:
        y = y + bias
    return y


def rope(x, positions, theta):
    """Half-split rotary embedding on x[T, heads, HD]   (src/operators/cpu/rope.cpp:36-56; cuda_rope.cu:8-34).

    freq_d = 1/theta^(2d/HD); a = pos*freq_d; (x[d], x[d+HD/2]) is rotated by a.
    """
    T, _, hd = x.shape
    half = hd // 2
    d = torch.arange(half, dtype=x.dtype)
    freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=x.dtype), 2.0 * d / hd)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]          # [T, half]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)


def attention(q, k, v, window=None):
    """Causal grouped-query attention of one whole sequence.

    q[T,NH,HD], k/v[T,NKV,HD]; head h reads kv head h // (NH/NKV); scale 1/sqrt(HD);
    keys j <= i only (src/inference/engines/generic_engine.cpp:625-627, 663-729;
    src/operators/cpu/attention.cpp:464-624; cuda_flash_attn.cu:154-248).
    ``window`` (not used by the reference's LLaMA path) keeps keys j > i - window.
    """
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty_like(q)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    mask = j <= i
    if window is not None:
        mask = mask & (j > i - window)
    for h in range(nh):
        kvh = h // group
        s = (q[:, h, :] @ k[:, kvh, :].t()) * scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kvh, :]
    return out


def swiglu(x, w_gate, w_up, w_down):
    """down( silu(x.Wg^T) * (x.Wu^T) ), silu(g) = g/(1+exp(-g))
    (src/inference/engines/generic_engine.cpp:776-780, 809; src/operators/cpu/elementwise.cpp:160-166)."""
    g = linear(x, w_gate)
    u = linear(x, w_up)
    m = g / (1.0 + torch.exp(-g)) * u
    return linear(m, w_down)


class PlainLlama:
    """Holds the tensors of a model folder under their file names and runs whole sequences."""

    def __init__(self, model_dir, dtype=torch.float64):
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
        self._setup(cfg, read_safetensors(os.path.join(model_dir, "model.safetensors")), dtype)

    @classmethod
    def from_tensors(cls, cfg, tensors, dtype=torch.float64):
        """cfg: dict with config.json keys; tensors: {file tensor name: numpy array}."""
        self = cls.__new__(cls)
        self._setup(dict(cfg), tensors, dtype)
        return self

    def _setup(self, cfg, raw, dtype):
        self.cfg = cfg
        self.w = {k: torch.from_numpy(v).to(dtype) for k, v in raw.items()}
        self.dtype = dtype
        c = self.cfg
        self.n_layers = c["num_hidden_layers"]
        self.nh = c["num_attention_heads"]
        self.nkv = c.get("num_key_value_heads", self.nh)
        self.hd = c.get("head_dim") or c["hidden_size"] // self.nh
        self.eps = c.get("rms_norm_eps", 1e-6)
        self.theta = c.get("rope_theta", 10000.0)
        self.tied = c.get("tie_word_embeddings", False)

    def layer(self, i, h, positions):
        """One decoder layer (src/inference/engines/generic_engine.cpp:916-1085):
        h1 = h + Wo.attn(rope(q),rope(k),v) of rmsnorm(h);  out = h1 + swiglu(rmsnorm(h1))."""
        w, p = self.w, f"model.layers.{i}."
        T = h.shape[0]
        x = rms_norm(h, w[p + "input_layernorm.weight"], self.eps)
        q = linear(x, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias"))
        k = linear(x, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias"))
        v = linear(x, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias"))
        q = rope(q.view(T, self.nh, self.hd), positions, self.theta)
        k = rope(k.view(T, self.nkv, self.hd), positions, self.theta)
        a = attention(q, k, v.view(T, self.nkv, self.hd))
        h1 = h + linear(a.reshape(T, self.nh * self.hd), w[p + "self_attn.o_proj.weight"])
        x2 = rms_norm(h1, w[p + "post_attention_layernorm.weight"], self.eps)
        return h1 + swiglu(x2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                           w[p + "mlp.down_proj.weight"])

    def logits(self, ids):
        """All T rows of logits for one request's tokens, positions 0..T-1
        (src/inference/engines/transformer_engine.cpp:445-522)."""
        ids = torch.as_tensor(ids, dtype=torch.long)
        positions = torch.arange(ids.numel())
        h = embedding(ids, self.w["model.embed_tokens.weight"])
        for i in range(self.n_layers):
            h = self.layer(i, h, positions)
        x = rms_norm(h, self.w["model.norm.weight"], self.eps)
        head = self.w["model.embed_tokens.weight"] if (self.tied and "lm_head.weight" not in self.w) \
            else self.w["lm_head.weight"]
        return linear(x, head)

    def generate_greedy(self, prompt, n_new):
        """Greedy generation by full recomputation; first maximum wins a tie
        (src/inference/generator.cpp:84-99, 235-293; sampler.cpp:137-142)."""
        ids = list(prompt)
        out = []
        for _ in range(n_new):
            lg = self.logits(ids)[-1]
            t = int(torch.argmax(lg))
            out.append(t)
            ids.append(t)
        return out
