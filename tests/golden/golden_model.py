"""Deterministic tiny LLaMA models for the golden comparison (numpy only).

Values come from a splitmix64 hash of (seed, tensor number, element number), so any
numpy version regenerates the same weights that the committed reference outputs were
computed from.
"""
import numpy as np

# Limits of the reference's CPU engine that shape these configs: hidden_size is a multiple of 32
# (its engine constructor re-quantizes the FP32 lm_head to Q8_0 blocks of 32 before the driver can
# put the FP32 tensor back, src/model/model_weights.cpp:40-67, and hangs on a ragged block), and
# vocab_size >= hidden_size (an embedding table with shape[0] < shape[1] is read as transposed,
# src/operators/cpu/embedding.cpp:248-260).
GOLDEN_CONFIGS = {
    # the first two differ in every size and option
    "mha_untied": dict(vocab_size=72, hidden_size=64, intermediate_size=88, num_hidden_layers=2,
                       num_attention_heads=5, num_key_value_heads=5, head_dim=8, rope_theta=10000.0,
                       rms_norm_eps=1e-5, tie_word_embeddings=False, attention_bias=False),
    "mqa_tied_bias": dict(vocab_size=128, hidden_size=96, intermediate_size=80, num_hidden_layers=3,
                          num_attention_heads=3, num_key_value_heads=1, head_dim=16, rope_theta=500000.0,
                          rms_norm_eps=1e-6, tie_word_embeddings=True, attention_bias=True),
    # 1 < kv heads < heads: with as many kv heads as heads, or with one, "h // group" and "h % kv heads"
    # pick the same kv head; only a true group tells them apart (src/operators/cpu/attention.cpp:464).
    # A large eps, so that the reference's use of it shows in the logits as well.
    "gqa_6_2_bias": dict(vocab_size=100, hidden_size=64, intermediate_size=72, num_hidden_layers=2,
                         num_attention_heads=6, num_key_value_heads=2, head_dim=8, rope_theta=30000.0,
                         rms_norm_eps=1e-2, tie_word_embeddings=False, attention_bias=True),
}
# steps of (start_pos, tokens): a prefill and then single tokens, as the reference's own
# incremental tests do (tests/test_operators.py:80-98)
GOLDEN_STEPS = {
    "mha_untied": [(0, [3, 70, 11, 25, 8, 41]), (6, [17]), (7, [2])],
    "gqa_6_2_bias": [(0, [9, 99, 4, 57, 23, 0, 61]), (7, [12]), (8, [88]), (9, [30])],
    "mqa_tied_bias": [(0, [5, 9, 127, 0, 31]), (5, [44]), (6, [7]), (7, [7])],
}


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15))
    z = x
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def hashed_normal(seed, tensor_no, n, std):
    """n float32 values ~ N(0, std) by Box-Muller over two hashed uniforms."""
    with np.errstate(over="ignore"):
        i = np.arange(n, dtype=np.uint64)
        base = _splitmix64(np.uint64(seed) * np.uint64(0x100000001B3) + np.uint64(tensor_no))
        a = _splitmix64(base + np.uint64(2) * i)
        b = _splitmix64(base + np.uint64(2) * i + np.uint64(1))
    u1 = ((a >> np.uint64(11)).astype(np.float64) + 1.0) / 9007199254740993.0
    u2 = (b >> np.uint64(11)).astype(np.float64) / 9007199254740992.0
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2) * std).astype(np.float32)


def golden_tensors(cfg, seed):
    """{HF tensor name: float32 array} in a fixed order (python dicts keep insertion order)."""
    V, H, I = cfg["vocab_size"], cfg["hidden_size"], cfg["intermediate_size"]
    NH, NKV, HD = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    t = {}
    no = [0]

    def mat(name, shape, std=0.08, mean=0.0):
        n = int(np.prod(shape))
        t[name] = (hashed_normal(seed, no[0], n, std) + np.float32(mean)).reshape(shape)
        no[0] += 1

    mat("model.embed_tokens.weight", (V, H), 0.5)
    mat("model.norm.weight", (H,), 0.1, 1.0)
    if not cfg["tie_word_embeddings"]:
        mat("lm_head.weight", (V, H), 0.2)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        mat(p + "input_layernorm.weight", (H,), 0.1, 1.0)
        mat(p + "self_attn.q_proj.weight", (NH * HD, H), 0.3)
        mat(p + "self_attn.k_proj.weight", (NKV * HD, H), 0.3)
        mat(p + "self_attn.v_proj.weight", (NKV * HD, H), 0.2)
        if cfg["attention_bias"]:
            mat(p + "self_attn.q_proj.bias", (NH * HD,), 0.2)
            mat(p + "self_attn.k_proj.bias", (NKV * HD,), 0.2)
            mat(p + "self_attn.v_proj.bias", (NKV * HD,), 0.2)
        mat(p + "self_attn.o_proj.weight", (H, NH * HD), 0.2)
        mat(p + "post_attention_layernorm.weight", (H,), 0.1, 1.0)
        mat(p + "mlp.gate_proj.weight", (I, H), 0.2)
        mat(p + "mlp.up_proj.weight", (I, H), 0.2)
        mat(p + "mlp.down_proj.weight", (H, I), 0.2)
    return t
