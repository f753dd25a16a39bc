"""Shared test helpers: seeded synthetic layers built once on the host (numpy + the oracle's quantizer port) and
mirrored onto the GPU, and the error metrics the parity tests use."""
import numpy as np

import oracle

BF16_ULP = 2.0 ** -7  # the largest relative size of one BF16 step (just above a power of two; 8 significand bits)


def rel_err_rows(y, ref):
    """max |y - ref| / max |ref| per row: the layer tolerance is stated against the row's largest magnitude, since an
    elementwise relative error is ill-posed near zeros."""
    y = np.asarray(y, np.float64).reshape(-1, y.shape[-1])
    ref = np.asarray(ref, np.float64).reshape(-1, ref.shape[-1])
    den = np.maximum(np.abs(ref).max(axis=1), 1e-30)
    return (np.abs(y - ref).max(axis=1) / den).max()


def bf16_rows_close(y, ref, tol):
    """BF16 outputs: |y - ref| <= tol * max|ref| of the row + one BF16 step of the reference element (the two sides may
    round a near-tie differently). Returns the worst excess ratio (<= 1 passes)."""
    y = np.asarray(y, np.float64).reshape(-1, y.shape[-1])
    ref = np.asarray(ref, np.float64).reshape(-1, ref.shape[-1])
    rowmax = np.maximum(np.abs(ref).max(axis=1, keepdims=True), 1e-30)
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref), 1e-30))) - 7)
    return (np.abs(y - ref) / (tol * rowmax + ulp)).max()


def to_np_act(t):
    """torch float32 / bfloat16 CUDA tensor -> numpy float32 / uint16 bits."""
    import torch

    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def to_torch_act(a, device="cuda"):
    import torch

    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(device).view(torch.bfloat16)
    return torch.from_numpy(a).to(device)


def randn_act(rng, shape, act, sigma=1.0):
    x = (rng.standard_normal(shape) * sigma).astype(np.float32)
    return x if act == oracle.F32 else oracle.f32_to_bf16(x)


def quantized(rng, bits, N, K, G, sigma=0.02):
    w = (rng.standard_normal((N, K)) * sigma).astype(np.float32)
    return oracle.quantize(bits, w, G)


def upload(qw):
    from strixite_b200 import kernels as K

    return K.QWeight.upload(qw.bits, qw.N, qw.K, qw.G, qw.q, qw.scale, qw.minv)


def upload_stack(st):
    """oracle.ExpertStack -> QWeight (uniform) or QMixStack (per-expert formats) on the device."""
    import torch

    from strixite_b200 import kernels as K

    if st.bits_tab is None:
        return K.QWeight.upload(st.bits, st.E * st.N, st.K, st.G, st.q, st.scale, st.minv)
    return K.QMixStack(st.E, st.N, st.K, st.G, torch.from_numpy(st.q).cuda(), torch.from_numpy(st.scale.view(np.int16)).cuda(),
                       torch.from_numpy(st.minv.view(np.int16)).cuda(), torch.from_numpy(st.bits_tab).cuda(),
                       torch.from_numpy(st.q_off).cuda())


def make_stack(rng, E, N, K, G, bits=4, mix=None, sigma=0.02):
    """Uniform stack in `bits`, or with mix = probabilities for (4, 5, 6, 8) a seeded format per expert."""
    if mix is None:
        return oracle.ExpertStack.from_weight(quantized(rng, bits, E * N, K, G, sigma), E)
    fmts = rng.choice([4, 5, 6, 8], size=E, p=mix)
    return oracle.ExpertStack.from_mixed([quantized(rng, int(b), N, K, G, sigma) for b in fmts])


def make_layer(seed, d, I, E, k, G=128, router="f32", shared="stacked", shared_coef="sigmoid", expert_bits=4, mix=None, bias_sigma=None,
               shared_bits=8, shared_G=64):
    """A seeded MoE layer in the oracle's dict form (see oracle.moe_layer)."""
    rng = np.random.default_rng(seed)
    gated = shared is not None and shared_coef == "sigmoid"
    R = E + (1 if gated else 0)
    rw = (rng.standard_normal((R, d)) * 0.02).astype(np.float32)
    if router == "bf16":
        rw = oracle.f32_to_bf16(rw)
    elif router == "q8":
        rw = oracle.quantize(8, rw, 64)
    Es = E + (1 if shared == "stacked" else 0)
    L = dict(E=E, k=k, d=d, I=I, router=rw, shared=shared, shared_coef=shared_coef,
             gate_up=make_stack(rng, Es, 2 * I, d, G, expert_bits, mix), down=make_stack(rng, Es, d, I, G, expert_bits, mix))
    if shared == "separate":
        L["sh_gate_up"] = quantized(rng, shared_bits, 2 * I, d, shared_G)
        L["sh_down"] = quantized(rng, shared_bits, d, I, shared_G)
    if bias_sigma is not None:
        L["router_bias"] = (rng.standard_normal(E) * bias_sigma).astype(np.float32)
    return L


def gpu_layer(L, act, max_tokens, grouped_min_tokens=6, math=0, decode_impl=0):
    """The device twin of a make_layer() dict."""
    import torch

    import strixite_b200 as sb

    r = L["router"]
    if isinstance(r, oracle.QWeight):
        router = upload(r)
    elif r.dtype == np.uint16:
        router = torch.from_numpy(r.view(np.int16)).cuda().view(torch.bfloat16)
    else:
        router = torch.from_numpy(r).cuda()
    kw = {}
    if L.get("shared") == "separate":
        kw.update(sh_gate_up=upload(L["sh_gate_up"]), sh_down=upload(L["sh_down"]))
    if L.get("router_bias") is not None:
        kw["router_bias"] = torch.from_numpy(L["router_bias"]).cuda()
    return sb.MoeLayer(L["d"], L["I"], L["E"], L["k"], act, router, upload_stack(L["gate_up"]), upload_stack(L["down"]),
                       shared=L.get("shared"), shared_coef=L.get("shared_coef", "sigmoid"), max_tokens=max_tokens,
                       grouped_min_tokens=grouped_min_tokens, math=math, decode_impl=decode_impl, **kw)
