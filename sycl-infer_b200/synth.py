"""Seeded synthetic GGUF block tensors and activations.

No GGUF model file ships with this repository, so every test and benchmark
workload is generated here as raw block bytes with the value distributions the
benchmark configurations describe: superblock scales d/dmin = f16(|N(0, 0.01)|),
packed 6-bit sub-scales uniform (12 random bytes -> every unpacked scale/min is
uniform in 0..63), quants uniform over their code range, activations N(0, 1).
Rows are laid out exactly like a GGUF tensor: row r starts at r * row_bytes.
"""
import numpy as np

Q8_0, Q4_K, Q5_K, Q6_K, IQ4_XS = 8, 12, 13, 14, 23
TYPE_NAMES = {Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", IQ4_XS: "IQ4_XS"}
TYPE_IDS = {v: k for k, v in TYPE_NAMES.items()}
SUPERBLOCK_BYTES = {Q4_K: 144, Q5_K: 176, Q6_K: 210, IQ4_XS: 136, Q8_0: 8 * 34}


def row_bytes(qtype, K):
    """Bytes of one weight row of K values (K a multiple of 256)."""
    return SUPERBLOCK_BYTES[qtype] * (K // 256)


def _f16_scale(rng, n, sigma=0.01):
    return np.abs(rng.normal(0.0, sigma, n)).astype(np.float16).view(np.uint16)


def _put16(buf, col, v):
    buf[:, col] = (v & 0xFF).astype(np.uint8)
    buf[:, col + 1] = (v >> 8).astype(np.uint8)


def make_weight(qtype, n_rows, K, seed):
    """Raw block bytes of an [n_rows][K] tensor as a flat uint8 array."""
    assert K % 256 == 0
    rng = np.random.default_rng(seed)
    nsb = n_rows * (K // 256)
    if qtype == Q8_0:
        b = rng.integers(0, 256, (nsb * 8, 34), dtype=np.uint8)
        q = rng.integers(-127, 128, (nsb * 8, 32), dtype=np.int8)
        b[:, 2:] = q.view(np.uint8)
        _put16(b, 0, _f16_scale(rng, nsb * 8))
        return b.reshape(-1)
    b = rng.integers(0, 256, (nsb, SUPERBLOCK_BYTES[qtype]), dtype=np.uint8)
    if qtype in (Q4_K, Q5_K):
        _put16(b, 0, _f16_scale(rng, nsb))
        _put16(b, 2, _f16_scale(rng, nsb))
    elif qtype == Q6_K:
        b[:, 192:208] = rng.integers(-32, 32, (nsb, 16), dtype=np.int8).view(np.uint8)
        _put16(b, 208, _f16_scale(rng, nsb))
    elif qtype == IQ4_XS:
        _put16(b, 0, _f16_scale(rng, nsb))
    else:
        raise ValueError(f"unsupported ggml type {qtype}")
    return b.reshape(-1)


def make_activation(n_tok, K, seed):
    return np.random.default_rng(seed).normal(0.0, 1.0, (n_tok, K)).astype(np.float32)


def make_router_logits(n_tok, n_expert, seed):
    return np.random.default_rng(seed).normal(0.0, 1.0, (n_tok, n_expert)).astype(np.float32)


# Dense layer of the 27B-shaped model the benchmark names: hidden 5120, 40 query
# heads and 8 KV heads of dim 128, FFN 17408.  (name, type in the Q4_K_M mix, rows, K)
def dense_layer_shapes(mix="Q4_K_M", hidden=5120, n_head=40, n_kv=8, head_dim=128, n_ff=17408):
    q, kv = n_head * head_dim, n_kv * head_dim
    if mix == "Q4_K_M":
        t = dict(q=Q4_K, k=Q4_K, v=Q6_K, o=Q4_K, gate=Q4_K, up=Q4_K, down=Q6_K)
    else:
        t = {n: TYPE_IDS[mix] for n in ("q", "k", "v", "o", "gate", "up", "down")}
    return [("q", t["q"], q, hidden), ("k", t["k"], kv, hidden), ("v", t["v"], kv, hidden),
            ("o", t["o"], hidden, q), ("gate", t["gate"], n_ff, hidden), ("up", t["up"], n_ff, hidden),
            ("down", t["down"], hidden, n_ff)]


def layer_weight_bytes(mix="Q4_K_M", **kw):
    return sum(row_bytes(t, K) * n for _, t, n, K in dense_layer_shapes(mix, **kw))
