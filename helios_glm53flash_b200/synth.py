"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

Inputs are drawn in fp32 from numpy's counter-based Philox generator (seed 0 unless stated) and
then cast, so the same tensors can be rebuilt on any machine without a dataset or checkpoint.
Everything is returned as numpy arrays; 16-bit float tensors are uint16 bit patterns.
"""
import numpy as np


def rng(seed=0):
    return np.random.Generator(np.random.Philox(seed))


def f32_to_bf16_bits(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_f16_bits(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def f16_bits_to_f32(b):
    return np.asarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)


def _softplus(x):
    return np.logaddexp(0.0, x)


def kda_inputs(seqlen, heads=32, dim=128, bsz=1, seed=0, normalise=True, g_scale=1.0):
    """KDA recurrence inputs of benchmark configs 0/1: q,k ~ N(0,1) L2-normalised per (token, head),
    v ~ N(0,1), beta = sigmoid(N(0,1)), log-decay g = -softplus(N(0,1)) per (token, head, channel).
    Returns dict(mixed_qkv bf16 bits [bsz][T][3*H*D], g f32 [bsz][T][H][D], beta bf16 bits [bsz][T][H])."""
    r = rng(seed)
    q = r.standard_normal((bsz, seqlen, heads, dim), dtype=np.float32)
    k = r.standard_normal((bsz, seqlen, heads, dim), dtype=np.float32)
    v = r.standard_normal((bsz, seqlen, heads, dim), dtype=np.float32)
    if normalise:
        q /= np.linalg.norm(q, axis=-1, keepdims=True)
        k /= np.linalg.norm(k, axis=-1, keepdims=True)
    beta = 1.0 / (1.0 + np.exp(-r.standard_normal((bsz, seqlen, heads), dtype=np.float32)))
    g = (-g_scale * _softplus(r.standard_normal((bsz, seqlen, heads, dim), dtype=np.float32))).astype(np.float32)
    mixed = np.concatenate([q.reshape(bsz, seqlen, -1), k.reshape(bsz, seqlen, -1),
                            v.reshape(bsz, seqlen, -1)], axis=-1)
    return {"mixed_qkv": f32_to_bf16_bits(mixed), "g": g, "beta": f32_to_bf16_bits(beta)}


def kda_gates(seqlen, heads=32, dim=128, bsz=1, seed=0):
    """only the gate tensors of kda_inputs (same distributions): g f32 [bsz][T][H][D], beta bf16 bits"""
    r = rng(seed + 505)
    beta = 1.0 / (1.0 + np.exp(-r.standard_normal((bsz, seqlen, heads), dtype=np.float32)))
    g = -_softplus(r.standard_normal((bsz, seqlen, heads, dim), dtype=np.float32))
    return {"g": g.astype(np.float32), "beta": f32_to_bf16_bits(beta)}


def kda_raw_gates(seqlen, heads=32, dim=128, seed=0):
    """Inputs of the gate preparation: raw gate projection f [T][H][D] ~ N(0,1), raw beta logit b [T][H] ~ N(0,1),
    dt_bias [H][D] ~ N(0,0.5), a_log [H] ~ U(log 0.5, log 4); the model's lower bound is -5."""
    r = rng(seed + 606)
    return {"f": r.standard_normal((seqlen, heads, dim), dtype=np.float32),
            "b": r.standard_normal((seqlen, heads), dtype=np.float32),
            "dt_bias": (0.5 * r.standard_normal((heads, dim), dtype=np.float32)).astype(np.float32),
            "a_log": r.uniform(np.log(0.5), np.log(4.0), heads).astype(np.float32),
            "lower_bound": -5.0}


def conv_inputs(seqlen, dim, bsz=1, K=4, seed=0):
    """Short-conv inputs: x ~ N(0,1) channel-major [bsz][dim][T], weights ~ N(0,0.1) [dim][K],
    previous window state ~ N(0,1) [bsz][dim][K]."""
    r = rng(seed + 101)
    x = r.standard_normal((bsz, dim, seqlen), dtype=np.float32)
    w = (0.1 * r.standard_normal((dim, K), dtype=np.float32)).astype(np.float32)
    st = r.standard_normal((bsz, dim, K), dtype=np.float32)
    return {"x": f32_to_bf16_bits(x), "weight": f32_to_bf16_bits(w), "state": f32_to_bf16_bits(st)}


def mla_inputs(cache_len, m=1, heads=64, seed=0, cache_std=1.0):
    """Absorbed-MLA inputs of config 2: latent cache [L][512] ~ N(0,1) fp16, absorbed queries
    [m][heads][512] ~ N(0,1) fp16."""
    r = rng(seed + 202)
    ckv = (cache_std * r.standard_normal((cache_len, 512), dtype=np.float32)).astype(np.float32)
    q = r.standard_normal((m, heads, 512), dtype=np.float32)
    return {"ckv": f32_to_f16_bits(ckv), "q_lat": f32_to_f16_bits(q)}


def indexer_inputs(npools, m=1, heads=32, seed=0, bf16=False):
    """Indexer inputs of config 3: pooled keys [npools][128] ~ N(0,1), queries [m][32][128] ~ N(0,1),
    head weights [m][32] ~ N(0,1); fp16 (reference dtype) or bf16 (config dtype) bit patterns."""
    r = rng(seed + 303)
    pk = r.standard_normal((npools, 128), dtype=np.float32)
    q = r.standard_normal((m, heads, 128), dtype=np.float32)
    w = r.standard_normal((m, heads), dtype=np.float32)
    cast = f32_to_bf16_bits if bf16 else f32_to_f16_bits
    return {"pool_k": cast(pk), "q_idx": cast(q), "w": cast(w)}


def shard_range(n, rank, world):
    """Contiguous [begin, end) of n units owned by `rank` of `world` (head / sequence sharding)."""
    base, rem = divmod(n, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)
