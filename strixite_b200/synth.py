"""Seeded synthetic MoE layers built directly on the device: FP32 N(0, sigma) weights drawn chunk by chunk with a
seeded torch generator and packed by the device quantizer (bit-identical to the host quantizer), so that layers of the
benchmark's full size (hundreds of MB to GB of packed weights per layer) never exist in FP32 as a whole.

Stands in for converted checkpoints, which are not available offline. Shapes follow the benchmark configurations:
hidden d, intermediate I, E routed experts (+1 shared), top-k.
"""
import numpy as np
import torch

from . import kernels as K
from .layer import MoeLayer

_CHUNK_ELEMS = 1 << 27  # FP32 elements drawn per chunk (512 MB)


def _gen(seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def quantized_normal(seed, bits, N, Kdim, G, sigma=0.02, device="cuda", out=None, row0=0):
    """QWeight [N, K] of N(0, sigma) weights, drawn and packed in row chunks."""
    g = _gen(seed, device)
    qw = K.QWeight.empty(bits, N, Kdim, G, device) if out is None else out
    rows_per = max(1, _CHUNK_ELEMS // Kdim)
    for r in range(0, N, rows_per):
        n = min(rows_per, N - r)
        w = torch.randn((n, Kdim), generator=g, device=device, dtype=torch.float32) * sigma
        K.QWeight.quantize_device(w, bits, G, out=qw, row0=row0 + r)
    return qw


def mixed_stack(seed, E, N, Kdim, G, probs, sigma=0.02, device="cuda"):
    """QMixStack of E experts [N, K] each, formats drawn from (4, 5, 6, 8) with `probs` by a seeded numpy generator."""
    rng = np.random.default_rng(seed)
    bits = rng.choice([4, 5, 6, 8], size=E, p=probs).astype(np.uint8)
    st = K.QMixStack.empty(bits, N, Kdim, G, device)
    off, _ = K.QMixStack.layout(bits, N, Kdim)
    g = _gen(seed + 1, device)
    for e in range(E):
        w = torch.randn((N, Kdim), generator=g, device=device, dtype=torch.float32) * sigma
        K.QWeight.quantize_device(w, int(bits[e]), G, out=st.expert(e, bits, off))
    return st, bits


def zipf_bias(seed, E, s=1.1):
    """Router bias b_e = log p_e with p_e proportional to rank(e)^-s, ranks assigned by a seeded permutation."""
    rng = np.random.default_rng(seed)
    rank = rng.permutation(E) + 1
    p = rank.astype(np.float64) ** -s
    p /= p.sum()
    return np.log(p).astype(np.float32)


def make_layer(seed, d, I, E, k, act, G=128, router="f32", shared="stacked", shared_coef="sigmoid", expert_bits=4, mix=None,
               bias=None, shared_bits=8, shared_G=64, max_tokens=8, grouped_min_tokens=6, math=K.MoeMath.F32, device="cuda",
               decode_impl=0, tensor_min_tokens=0):
    """A seeded layer on the device. router: 'f32' | 'bf16' | 'q8'. mix: probabilities for per-expert (4, 5, 6, 8)-bit
    formats, or None for a uniform `expert_bits` stack. bias: None or a float32 numpy [E]. decode_impl: 0 = the fused
    single-kernel path for up to 8 tokens, 1 = the per-function kernels."""
    gated = shared is not None and shared_coef == "sigmoid"
    R = E + (1 if gated else 0)
    g = _gen(seed, device)
    rw = torch.randn((R, d), generator=g, device=device, dtype=torch.float32) * 0.02
    if router == "bf16":
        rw = rw.to(torch.bfloat16)
    elif router == "q8":
        rw, _ = K.QWeight.quantize_device(rw, 8, 64)
    Es = E + (1 if shared == "stacked" else 0)
    info = {}
    if mix is None:
        gate_up = quantized_normal(seed + 1, expert_bits, Es * 2 * I, d, G, device=device)
        down = quantized_normal(seed + 2, expert_bits, Es * d, I, G, device=device)
    else:
        gate_up, info["gate_up_bits"] = mixed_stack(seed + 1, Es, 2 * I, d, G, mix, device=device)
        down, info["down_bits"] = mixed_stack(seed + 3, Es, d, I, G, mix, device=device)
    kw = {}
    if shared == "separate":
        kw["sh_gate_up"] = quantized_normal(seed + 5, shared_bits, 2 * I, d, shared_G, device=device)
        kw["sh_down"] = quantized_normal(seed + 6, shared_bits, d, I, shared_G, device=device)
    if bias is not None:
        kw["router_bias"] = torch.from_numpy(np.ascontiguousarray(bias, np.float32)).to(device)
    layer = MoeLayer(d, I, E, k, act, rw, gate_up, down, shared=shared, shared_coef=shared_coef, max_tokens=max_tokens,
                     grouped_min_tokens=grouped_min_tokens, math=math, decode_impl=decode_impl, tensor_min_tokens=tensor_min_tokens, **kw)
    layer.weights = dict(router=rw, gate_up=gate_up, down=down, **kw)
    layer.info = info
    return layer
