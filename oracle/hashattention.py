"""HashAttention signatures and scores
(research_attention/maskers/fixed/implementations/hashattention_top_k.py)."""

import math

import numpy as np

from .bf16 import bits_of, from_bits, round_bf16, round_to

_TABLES = {}


def activation_table(name: str) -> np.ndarray:
    """uint16[65536]: bf16 bits of x -> bf16 bits of act(x), evaluated in float64 and
    rounded through float32 to bfloat16 (the value a float32 kernel such as
    torch.nn.functional.silu on a bf16 tensor rounds to)."""
    if name in _TABLES:
        return _TABLES[name]
    x = from_bits(np.arange(65536, dtype=np.uint32).astype(np.uint16)).astype(np.float64)
    with np.errstate(over="ignore", invalid="ignore"):
        if name == "relu":
            y = np.maximum(x, 0.0)
        elif name == "silu":
            y = x / (1.0 + np.exp(-x))
        elif name == "gelu":
            y = 0.5 * x * (1.0 + np.vectorize(math.erf)(x / math.sqrt(2.0)))
        elif name == "tanh":
            y = np.tanh(x)
        else:
            raise ValueError(f"Unsupported activation function: {name}")
    y = np.where(np.isnan(x), x, y)
    t = bits_of(round_bf16(y.astype(np.float32)))
    t[np.isnan(y)] = 0x7FC0
    _TABLES[name] = t
    return t


def _activate(y: np.ndarray, name: str, dtype: str) -> np.ndarray:
    if dtype == "bf16":
        return from_bits(activation_table(name)[bits_of(y)])
    y = y.astype(np.float32)
    if name == "relu":
        return np.maximum(y, np.float32(0))
    if name == "silu":
        return (y / (np.float32(1) + np.exp(-y))).astype(np.float32)
    if name == "gelu":
        return (np.float32(0.5) * y * (np.float32(1) + np.vectorize(math.erf)(y / math.sqrt(2.0)))).astype(np.float32)
    if name == "tanh":
        return np.tanh(y).astype(np.float32)
    raise ValueError(f"Unsupported activation function: {name}")


def mlp_outputs(x, mats, biases, act: str, dtype: str) -> np.ndarray:
    """_get_signatures before the sign (:203-238): per-head MLP
    `einsum("bhsd,hde->bhse") + bias`, activation between layers, none after the last.

    Summation order fixed here: one fp32 accumulator per output, input channels
    in ascending order, fused multiply-add; the sum, the bias add and the
    activation are each rounded to `dtype`.
    x [B,H,n,D]; mats[l] [H,in,out]; biases[l] [H,out].
    """
    h = np.asarray(x, np.float32)
    for l, (W, b) in enumerate(zip(mats, biases)):
        W = np.asarray(W, np.float32)
        acc = np.zeros(h.shape[:-1] + (W.shape[-1],), np.float32)
        for d in range(W.shape[1]):
            prod = h[..., d:d + 1].astype(np.float64) * W[None, :, None, d, :].astype(np.float64)
            acc = (acc.astype(np.float64) + prod).astype(np.float32)
        y = round_to(acc, dtype)
        y = round_to(y + np.asarray(b, np.float32)[None, :, None, :], dtype)
        if l < len(mats) - 1:
            y = _activate(y, act, dtype)
        h = y
    return h


def signatures_blas(x, mats, biases, act: str, dtype: str) -> np.ndarray:
    """Same MLP with float32 BLAS products (summation order left to the BLAS, as in the
    reference).  Used only to set up timing runs at sizes where the ordered loop of
    `mlp_outputs` is too slow; parity checks use `signatures`."""
    h = np.asarray(x, np.float32)
    for l, (W, b) in enumerate(zip(mats, biases)):
        Wf = np.asarray(W, np.float32)
        y = np.empty(h.shape[:-1] + (Wf.shape[-1],), np.float32)
        for hh in range(Wf.shape[0]):
            y[:, hh] = h[:, hh] @ Wf[hh]
        y = round_to(y, dtype)
        y = round_to(y + np.asarray(b, np.float32)[None, :, None, :], dtype)
        if l < len(mats) - 1:
            y = _activate(y, act, dtype)
        h = y
    return pack_signs(h)


def pack_signs(y: np.ndarray) -> np.ndarray:
    """bit e = 1 where output e > 0 (sign == +1); uint32 per vector."""
    bits = (y > 0).astype(np.uint32)
    weights = (np.uint32(1) << np.arange(y.shape[-1], dtype=np.uint32))
    return (bits * weights).sum(axis=-1).astype(np.uint32)


def signatures(x, mats, biases, act: str, dtype: str) -> np.ndarray:
    return pack_signs(mlp_outputs(x, mats, biases, act, dtype))


def scores(qcodes: np.ndarray, kcodes: np.ndarray, nbits: int, dtype: str,
           attention_mask=None) -> np.ndarray:
    """_compute_hashattention_score (:343-371) on packed signatures:
    dot of +-1 vectors = nbits - 2 * hamming; + attention mask, rounded in `dtype`.
    qcodes [B,H,Sq], kcodes [B,H,S] -> [B,H,Sq,S] float32."""
    ham = np.bitwise_count(qcodes[..., :, None] ^ kcodes[..., None, :]).astype(np.float32)
    s = np.float32(nbits) - np.float32(2) * ham
    if attention_mask is not None:
        s = round_to(s + np.asarray(attention_mask, np.float32)[..., : s.shape[-1]], dtype)
    return s
