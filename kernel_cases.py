"""Runs ONE kernel at a named workload a few times: the small, self-contained cases that profiles/ are
captured from (`ncu ... python kernel_cases.py <case>`), each also timed with CUDA events.

Cases use the layer sizes of the TinyLlama-1.1B shape: hidden 2048, 32 heads / 4 kv heads of 64, feed-forward 5632.
"""
import sys
from types import SimpleNamespace

import torch

from forge_b200.kernels import (decode_attention_fused, gemm_sm100, gemm_sm100_qkv_rope, paged_attention, paged_attention_mma,
                                rope_table)

DEV = "cuda:0"
H, I, NH, NKV, HD, PS = 2048, 5632, 32, 4, 64, 16


def _bf16(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def _attention_inputs(reqs, NH=NH, NKV=NKV, HD=HD):
    """reqs: [(context_before, q_len)]; pages laid out in order."""
    pages = sum(-(-(c + q) // PS) for c, q in reqs)
    max_pages = max(-(-(c + q) // PS) for c, q in reqs)
    table = torch.zeros(len(reqs), max_pages, dtype=torch.int32)
    q_start, nxt = [0], 0
    for s, (c, q) in enumerate(reqs):
        n = -(-(c + q) // PS)
        table[s, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
        nxt += n
        q_start.append(q_start[-1] + q)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    batch = SimpleNamespace(num_requests=len(reqs), host_q_start=q_start, host_context_before=[c for c, _ in reqs],
                            q_start=i32(q_start), context_before=i32([c for c, _ in reqs]), attention_plan={})
    return (_bf16(q_start[-1], NH * HD), _bf16(pages, 2, NKV, PS, HD), SimpleNamespace(block_table=table.to(DEV)), batch)


def case(name):
    if name == "gemm_decode_gateup":         # 8 tokens x [11264, 2048] weights, SwiGLU epilogue: 46 MB streamed
        x, w = _bf16(8, H), _bf16(2 * I, H, scale=0.02)
        return (lambda: gemm_sm100(x, w, epilogue="swiglu")), w.numel() * 2, 2 * 8 * w.numel()
    if name == "gemm_decode_down":           # 8 tokens x [2048, 5632], residual accumulate, K cut over a cluster
        x, w, r = _bf16(8, I), _bf16(H, I, scale=0.02), torch.zeros(8, H, device=DEV)
        return (lambda: gemm_sm100(x, w, accumulate_into=r)), w.numel() * 2, 2 * 8 * w.numel()
    if name == "gemm_decode_lmhead":         # 8 tokens x [32000, 2048]: 250 row tiles, dealt out evenly (stream-K)
        x, w = _bf16(8, H), _bf16(32000, H, scale=0.02)
        return (lambda: gemm_sm100(x, w)), w.numel() * 2, 2 * 8 * w.numel()
    if name == "gemm_prefill_qkv":           # 2048 tokens x [2560, 2048]: tiles of 128 x 160 fill two waves
        x, w = _bf16(2048, H), _bf16((NH + 2 * NKV) * HD, H, scale=0.02)
        return (lambda: gemm_sm100(x, w)), (x.numel() + w.numel()) * 2 + 2048 * w.shape[0] * 4, 2 * 2048 * w.numel()
    if name == "gemm_prefill_gateup":        # 2048 tokens x [11264, 2048], SwiGLU epilogue: 94.5 GFLOP
        x, w = _bf16(2048, H), _bf16(2 * I, H, scale=0.02)
        return (lambda: gemm_sm100(x, w, epilogue="swiglu")), (x.numel() + w.numel() + 2048 * I) * 2, 2 * 2048 * w.numel()
    if name == "gemm_prefill_down":          # 2048 tokens x [2048, 5632], residual accumulate: 47.2 GFLOP
        x, w, r = _bf16(2048, I), _bf16(H, I, scale=0.02), torch.zeros(2048, H, device=DEV)
        return (lambda: gemm_sm100(x, w, accumulate_into=r)), (x.numel() + w.numel()) * 2 + r.numel() * 8, 2 * 2048 * w.numel()
    if name == "attention_decode":           # 64 requests, 1024 cached tokens each, one new token: 67 MB of K/V
        q, kv, g, b = _attention_inputs([(1023, 1)] * 64)
        return (lambda: paged_attention_mma(q, kv, g, b, NH, NKV, HD, PS)), 64 * 1024 * 2 * NKV * HD * 2, 4 * 64 * 1024 * NH * HD
    if name == "attention_decode_fused":     # the same decode step as one kernel: rotary + cache write + attention
        q, kv, g, b = _attention_inputs([(1023, 1)] * 64)
        qkv = torch.randn(64, (NH + 2 * NKV) * HD, device=DEV)
        pos = torch.full((64,), 1023, dtype=torch.int32, device=DEV)
        slots = (g.block_table[:, 1023 // PS] * PS + 1023 % PS).to(torch.int32).contiguous()
        return (lambda: decode_attention_fused(qkv, kv, g.block_table, pos, slots, NH, NKV, HD, PS, 1e4)), \
            64 * 1024 * 2 * NKV * HD * 2, 4 * 64 * 1024 * NH * HD
    if name == "attention_decode_stream":    # 32 requests x 8192 cached tokens through the TMA ring: 268 MB of keys and values
        from forge_b200.kernels import decode_attention_stream
        ctx, S, ps = 8192, 32, 64
        pages_per = ctx // ps + 1
        table = torch.arange(S * pages_per, dtype=torch.int32, device=DEV).reshape(S, pages_per)
        kv = _bf16(S * pages_per, 2, NKV, ps, HD)
        qkv = torch.randn(S, (NH + 2 * NKV) * HD, device=DEV)
        pos = torch.full((S,), ctx, dtype=torch.int32, device=DEV)
        slots = (table[:, ctx // ps] * ps + ctx % ps).to(torch.int32)
        return (lambda: decode_attention_stream(qkv, kv, table, pos, slots, NH, NKV, HD, ps, 1e4, max_context=ctx + 1)), \
            S * ctx * 2 * NKV * HD * 2, 4 * S * ctx * NH * HD
    if name == "attention_prefill":          # one request, 2048 tokens, causal: 17.2 GFLOP
        q, kv, g, b = _attention_inputs([(0, 2048)])
        return (lambda: paged_attention(q, kv, g, b, NH, NKV, HD, PS)), 0, 2 * 2048 * 2048 * NH * HD
    if name == "attention_prefill_hd128":    # the Llama-3-8B heads: 32 / 8 kv heads of 128, one request of 2048 tokens: 34.4 GFLOP
        q, kv, g, b = _attention_inputs([(0, 2048)], 32, 8, 128)
        return (lambda: paged_attention(q, kv, g, b, 32, 8, 128, PS)), 0, 2 * 2048 * 2048 * 32 * 128
    if name == "attention_prefill_shared_keys":     # 256 new tokens on 20,000 cached: 16 tiles x 4 kv heads, each tile's keys shared out among 4 CTAs
        q, kv, g, b = _attention_inputs([(20000, 256)])
        return (lambda: paged_attention(q, kv, g, b, NH, NKV, HD, PS)), 20256 * 2 * NKV * HD * 2, 4 * 256 * 20128 * NH * HD
    if name == "gemm_prefill_qkv_rope":      # 2048 tokens x [2560, 2048]; the epilogue rotates q, k and writes q (bf16) and the cache
        x, w = _bf16(2048, H), _bf16((NH + 2 * NKV) * HD, H, scale=0.02)
        pos = torch.arange(2048, dtype=torch.int32, device=DEV)
        table, kv = rope_table(pos, HD, 1e4, by_pair=True), _bf16(2048 // PS, 2, NKV, PS, HD)
        return (lambda: gemm_sm100_qkv_rope(x, w, None, table, pos, kv, NH, NKV, HD, PS)), \
            (x.numel() + w.numel()) * 2 + 2048 * w.shape[0] * 2, 2 * 2048 * w.numel()
    if name == "attention_prefill_mma":      # the same through the mma.sync kernel, for comparison
        q, kv, g, b = _attention_inputs([(0, 2048)])
        return (lambda: paged_attention_mma(q, kv, g, b, NH, NKV, HD, PS)), 0, 2 * 2048 * 2048 * NH * HD
    raise SystemExit(f"unknown case {name!r}; known: gemm_decode_gateup gemm_decode_down gemm_decode_lmhead gemm_prefill_qkv "
                     "gemm_prefill_gateup "
                     "gemm_prefill_qkv_rope gemm_prefill_down attention_decode attention_decode_fused attention_decode_stream attention_prefill "
                     "attention_prefill_hd128 attention_prefill_mma attention_prefill_shared_keys")


def main(argv):
    name = argv[1] if len(argv) > 1 else ""
    fn, nbytes, flops = case(name)
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        fn()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / 3 * 1e3
    print(f"{name}: {us:.1f} us per launch (3 launches back to back, warm L2), "
          f"{nbytes / us / 1e3:.0f} GB/s of algorithmic bytes, {flops / us / 1e6:.1f} TFLOP/s")


if __name__ == "__main__":
    main(sys.argv)
