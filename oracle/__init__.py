"""TEST INFRASTRUCTURE - NOT PRODUCT CODE.

ctypes doors onto the CPU checker libraries built by oracle/build.py:

  orc   liboracle.so        the double-accumulating restatement of strixite's MoE-FFN arithmetic
  fast  liboracle_fast.so   the timed multi-threaded CPU baseline
  ref   _ref/libstrix_formats_ref.so   the reference's own quantizers (None when not built)

Only tests/, the smoke check and the bench's CPU legs may import this package; the product package never does.
All arrays are numpy; activations are float32 (act = F32) or uint16 bf16 bits (act = BF16).
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
F32, BF16 = 0, 1

_i64, _i32, _int, _u32, _vp = C.c_int64, C.c_int32, C.c_int, C.c_uint32, C.c_void_p


def _load(name):
    p = os.path.join(HERE, name)
    return C.CDLL(p) if os.path.exists(p) else None


def _ensure_built():
    if not (os.path.exists(os.path.join(HERE, "liboracle.so")) and os.path.exists(os.path.join(HERE, "liboracle_fast.so"))):
        from . import build as _b

        _b.build()


_ensure_built()
orc = _load("liboracle.so")
fast = _load("liboracle_fast.so")
ref = _load(os.path.join("_ref", "libstrix_formats_ref.so"))
if ref is not None:
    ref.ref_last_error.restype = C.c_char_p
orc.orc_row_bytes.restype = _i64
orc.orc_row_bytes.argtypes = [_int, _i64]
orc.orc_route_workspace_ints.restype = _i64
orc.orc_route_workspace_ints.argtypes = [_i64, _i64, _i64]
orc.orc_f32_to_bf16.restype = C.c_uint16
orc.orc_f32_to_bf16.argtypes = [C.c_float]
orc.orc_bf16_to_f32.restype = C.c_float
orc.orc_bf16_to_f32.argtypes = [C.c_uint16]


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(_vp)


def act_of(a):
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.uint16:
        return BF16
    raise TypeError("activations must be float32 or uint16 (bf16 bits), got %s" % a.dtype)


def empty_act(shape, act):
    return np.empty(shape, np.float32 if act == F32 else np.uint16)


def f32_to_bf16(a):
    """RNE with NaN quieting, vectorized (formats/q4.cpp:14-20)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    nan = (u & 0x7F800000) == 0x7F800000
    r = ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    n = ((u >> 16) | np.where(u & 0x007FFFFF, 0x0040, 0)).astype(np.uint16)
    return np.where(nan, n, r).astype(np.uint16)


def bf16_to_f32(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_f32(a):
    return a if a.dtype == np.float32 else bf16_to_f32(a)


def row_bytes(bits, K):
    return int(orc.orc_row_bytes(bits, K))


class QWeight:
    """Host copy of a quantized matrix [N, K]: q [N * row_bytes] u8, scale/minv [N, K/G] bf16 bits."""

    def __init__(self, bits, N, K, G, q, scale, minv):
        self.bits, self.N, self.K, self.G, self.q, self.scale, self.minv = bits, N, K, G, q, scale, minv

    def nbytes(self):
        return self.q.nbytes + self.scale.nbytes + self.minv.nbytes


def _quantize(lib, fn, bits, w, G):
    w = np.ascontiguousarray(w, np.float32)
    N, K = w.shape
    q = np.zeros(N * row_bytes(bits, K), np.uint8)
    s = np.zeros((N, max(K // G, 1)), np.uint16)
    m = np.zeros((N, max(K // G, 1)), np.uint16)
    rc = getattr(lib, fn)(_int(bits), _p(w), _i64(N), _i64(K), _i64(G), _p(q), _p(s), _p(m))
    return rc, QWeight(bits, N, K, G, q, s, m)


def quantize(bits, w, G):
    rc, qw = _quantize(orc, "orc_quantize", bits, w, G)
    if rc != 0:
        raise ValueError("orc_quantize failed with code %d" % rc)
    return qw


def quantize_rc(bits, w, G):
    return _quantize(orc, "orc_quantize", bits, w, G)[0]


def ref_quantize(bits, w, G):
    rc, qw = _quantize(ref, "ref_quantize", bits, w, G)
    if rc != 0:
        raise ValueError(ref.ref_last_error().decode())
    return qw


def ref_to_chunk_major(w):
    """The reference's own to_chunk_major (formats/q4.cpp:101-119, formats/q8.cpp) through oracle/_ref."""
    q, sc, mn = np.empty_like(w.q), np.empty_like(w.scale), np.empty_like(w.minv)
    rc = ref.ref_to_chunk_major(_int(w.bits), _p(w.q), _p(w.scale), _p(w.minv), _i64(w.N), _i64(w.K), _i64(w.G), _p(q),
                                _p(sc), _p(mn))
    if rc != 0:
        raise RuntimeError(ref.ref_last_error().decode())
    return QWeight(w.bits, w.N, w.K, w.G, q, sc, mn)


def dequantize(qw, lib=None, fn="orc_dequantize"):
    out = np.empty((qw.N, qw.K), np.float32)
    rc = getattr(lib or orc, fn)(_int(qw.bits), _p(qw.q), _p(qw.scale), _p(qw.minv), _i64(qw.N), _i64(qw.K), _i64(qw.G), _p(out))
    if lib is not None and rc != 0:
        raise ValueError(ref.ref_last_error().decode())
    return out


def ref_dequantize(qw):
    return dequantize(qw, ref, "ref_dequantize")


def ref_q4_from_q8(q8, G4, threads=1):
    N, K = q8.N, q8.K
    q = np.zeros(N * K // 2, np.uint8)
    s = np.zeros((N, K // G4), np.uint16)
    m = np.zeros((N, K // G4), np.uint16)
    rc = ref.ref_q4_from_q8(_p(q8.q), _p(q8.scale), _p(q8.minv), _i64(N), _i64(K), _i64(q8.G), _i64(G4), _int(threads), _p(q), _p(s), _p(m))
    if rc != 0:
        raise ValueError(ref.ref_last_error().decode())
    return QWeight(4, N, K, G4, q, s, m)


class ExpertStack:
    """E experts of N rows each, [E*N, K]. Uniform format (bits) or per-expert formats (bits_tab [E] u8, q_off [E] i64
    byte offsets into q); scale/minv are always [E*N, K/G]."""

    def __init__(self, E, N, K, G, q, scale, minv, bits=4, bits_tab=None, q_off=None):
        self.E, self.N, self.K, self.G, self.q, self.scale, self.minv = E, N, K, G, q, scale, minv
        self.bits, self.bits_tab, self.q_off = bits, bits_tab, q_off

    @staticmethod
    def from_weight(qw, E):
        assert qw.N % E == 0
        return ExpertStack(E, qw.N // E, qw.K, qw.G, qw.q, qw.scale, qw.minv, bits=qw.bits)

    @staticmethod
    def from_mixed(parts):
        """parts: one QWeight [N, K] per expert, any mix of formats with equal N, K, G."""
        E, N, K, G = len(parts), parts[0].N, parts[0].K, parts[0].G
        off = np.zeros(E, np.int64)
        total = 0
        for e, p in enumerate(parts):
            assert (p.N, p.K, p.G) == (N, K, G)
            off[e] = total
            total += (p.q.nbytes + 255) // 256 * 256
        q = np.zeros(total, np.uint8)
        for e, p in enumerate(parts):
            q[off[e] : off[e] + p.q.nbytes] = p.q
        return ExpertStack(E, N, K, G, q, np.concatenate([p.scale for p in parts]), np.concatenate([p.minv for p in parts]),
                           bits=0, bits_tab=np.array([p.bits for p in parts], np.uint8), q_off=off)

    def nbytes_of(self, e):
        b = int(self.bits_tab[e]) if self.bits_tab is not None else self.bits
        return self.N * (row_bytes(b, self.K) + 4 * (self.K // self.G))

    def _args(self):
        return [_int(self.bits), _p(self.bits_tab), _p(self.q_off)]

    def _wargs(self):
        return [_p(self.q), _p(self.scale), _p(self.minv), _i64(self.E), _i64(self.N), _i64(self.K), _i64(self.G)]


def linear_q(x, qw, out_act=None, lib=None, fn="orc_linear_q"):
    act = act_of(x)
    out_act = act if out_act is None else out_act
    M = x.shape[0]
    y = empty_act((M, qw.N), out_act)
    getattr(lib or orc, fn)(_int(qw.bits), _p(x), _int(act), _p(qw.q), _p(qw.scale), _p(qw.minv), _i64(qw.N), _i64(qw.K),
                            _i64(qw.G), _p(y), _int(out_act), _i64(M))
    return y


def linear_w(x, w, out_act=None, lib=None, fn="orc_linear_w"):
    """w float32 [N, K] or uint16 bf16 bits [N, K]."""
    act = act_of(x)
    out_act = act if out_act is None else out_act
    M, (N, K) = x.shape[0], w.shape
    y = empty_act((M, N), out_act)
    getattr(lib or orc, fn)(_p(x), _int(act), _p(w), _int(act_of(w)), _p(y), _int(out_act), _i64(M), _i64(N), _i64(K))
    return y


def moe_router(logits, E, k, shared_col=None, shared_id=0, err=None):
    """logits [M, ld]; shared_col = column of the shared gate logit in the same array, or None."""
    act = act_of(logits)
    M, ld = logits.shape
    A = k + (1 if shared_col is not None else 0)
    ids = np.empty((M, A), np.int32)
    coef = np.empty((M, A), np.float32)
    err = np.zeros(3, np.uint32) if err is None else err
    sp = None
    if shared_col is not None:
        sp = _vp(logits.ctypes.data + shared_col * logits.itemsize)
    orc.orc_moe_router(_p(logits), _i64(ld), _i64(M), _i64(E), _i64(k), sp, _i64(ld), _i32(shared_id), _p(ids), _p(coef),
                       _int(act), _p(err))
    return ids, coef, err


def swiglu(gu, I):
    act = act_of(gu)
    rows = gu.size // (2 * I)
    h = empty_act((rows, I), act)
    orc.orc_swiglu(_p(gu), _p(h), _i64(rows), _i64(I), _int(act))
    return h


def experts_gather(x, st, ids, swiglu=False, err=None, use_fast=False):
    act = act_of(x)
    M, A = ids.shape
    out = st.N // 2 if swiglu else st.N
    y = empty_act((M, A, out), act)
    err = np.zeros(3, np.uint32) if err is None else err
    if use_fast:
        assert swiglu
        fast.orc_fast_experts_gather_swiglu(*st._args(), _p(x), *st._wargs(), _p(ids), _i64(M), _i64(A), _p(y), _int(act))
    else:
        orc.orc_experts_gather(*st._args(), _p(x), *st._wargs(), _p(ids), _i64(M), _i64(A), _p(y), _int(act), _p(err),
                               _int(1 if swiglu else 0))
    return y, err


def experts_combine(h, st, ids, coef, err=None, use_fast=False):
    act = act_of(h)
    M, A = ids.shape
    y = empty_act((M, st.N), act)
    err = np.zeros(3, np.uint32) if err is None else err
    if use_fast:
        fast.orc_fast_experts_combine(*st._args(), _p(h), *st._wargs(), _p(ids), _p(coef), _i64(M), _i64(A), _p(y), _int(act))
    else:
        orc.orc_experts_combine(*st._args(), _p(h), *st._wargs(), _p(ids), _p(coef), _i64(M), _i64(A), _p(y), _int(act), _p(err))
    return y, err


def route_workspace_ints(M, A, E):
    return int(orc.orc_route_workspace_ints(M, A, E))


def group_routes(ids, E, err=None):
    M, A = ids.shape
    ws = np.full(route_workspace_ints(M, A, E), -7, np.int32)
    err = np.zeros(3, np.uint32) if err is None else err
    orc.orc_group_routes(_p(ids), _i64(M), _i64(A), _i64(E), _p(ws), _p(err))
    return ws, err


def moe_shared_add(y, s, gate_logit, gate_col, gate_index, err=None):
    """y [M, N] updated in place; gate_logit float32 [M, ld], the gate at column gate_col."""
    act = act_of(y)
    M, N = y.shape
    err = np.zeros(3, np.uint32) if err is None else err
    gp = _vp(gate_logit.ctypes.data + 4 * gate_col)
    orc.orc_moe_shared_add(_p(y), _p(s), gp, _i64(gate_logit.shape[1]), _i64(M), _i64(N), _u32(gate_index), _int(act), _p(err))
    return err


def moe_shared_add_inject(y, s, gate_logit, gate_col, gate_index, x, w_in, err=None):
    act = act_of(y)
    M, N = y.shape
    H = w_in.shape[1]
    err = np.zeros(3, np.uint32) if err is None else err
    gp = _vp(gate_logit.ctypes.data + 4 * gate_col)
    orc.orc_moe_shared_add_inject(_p(y), _p(s), gp, _i64(gate_logit.shape[1]), _i64(M), _i64(N), _u32(gate_index), _p(x),
                                  _p(w_in), _i64(H), _int(act), _p(err))
    return err


def hc_inject(x, y, w_in):
    M, N = y.shape
    orc.orc_hc_inject(_p(x), _p(y), _p(w_in), _i64(M), _i64(N), _i64(w_in.shape[1]), _int(act_of(y)))


def hc_mix_down(x, w, H, d, r, inject, eps=1e-6):
    """kernels/hc.hpp:36-39: x [T, H*d] (float32 or bf16 bits), w QWeight [r (+ H), H*d] (4 or 8 bits, folded).
    Returns (h [T, r], w_in [T, H] or None, inv [T, H]) float32."""
    T = x.shape[0]
    assert w.bits in (4, 8) and w.K == H * d and w.N == r + (H if inject else 0)
    h = np.zeros((T, r), np.float32)
    w_in = np.zeros((T, H), np.float32) if inject else None
    inv = np.zeros((T, H), np.float32)
    orc.orc_hc_mix_down(_p(x), _int(w.bits), _p(w.q), _p(w.scale), _p(w.minv), _i64(w.G), _i64(T), _i64(H), _i64(d),
                        _i64(r), _int(1 if inject else 0), C.c_float(eps), _p(h), _p(w_in), _p(inv), _int(act_of(x)))
    return h, w_in, inv


def to_chunk_major(w):
    """formats/q4.hpp:41-55 / formats/q8.hpp:37-46: the chunk-major copy of a 4- or 8-bit QWeight."""
    assert w.bits in (4, 8) and w.K % 32 == 0
    q, sc, mn = np.empty_like(w.q), np.empty_like(w.scale), np.empty_like(w.minv)
    orc.orc_to_chunk_major(_int(w.bits), _p(w.q), _p(w.scale), _p(w.minv), _i64(w.N), _i64(w.K), _i64(w.G), _p(q), _p(sc),
                           _p(mn))
    return QWeight(w.bits, w.N, w.K, w.G, q, sc, mn)


def hc_mix_up(h, w_up_cm, x, norm_w, inv, H, d):
    """kernels/hc.hpp:47-50: h [T, r] float32, w_up_cm the CHUNK-major QWeight [H*d, r], x [T, H*d], norm_w [H*d],
    inv [T, H]. Returns u [T, d] in x's dtype."""
    T, r = h.shape
    assert w_up_cm.bits in (4, 8) and w_up_cm.N == H * d and w_up_cm.K == r and r % 32 == 0
    u = np.zeros((T, d), x.dtype)
    orc.orc_hc_mix_up(_p(h), _int(w_up_cm.bits), _p(w_up_cm.q), _p(w_up_cm.scale), _p(w_up_cm.minv), _i64(w_up_cm.G),
                      _i64(r), _p(x), _p(norm_w), _p(inv), _i64(T), _i64(H), _i64(d), _p(u), _int(act_of(x)))
    return u


def residual_add(x, y):
    orc.orc_residual_add(_p(x), _p(y), _i64(x.size), _int(act_of(x)))


def fast_threads():
    return int(fast.orc_fast_threads())


def moe_layer(x, L, use_fast=False):
    """The MoE sublayer as strixite's runtime drives it (runtime/qwen4exp.cpp:1126-1186), from the pieces above.

    L: dict with
      E, k                         routed experts, top-k
      router                       float32 / bf16-bits ndarray [R, d] or QWeight [R, d]; R = E + 1 when the shared
                                   expert is gated (row E = its gate), else E
      router_bias                  optional float32 [E] added to the routed logits before selection (harness-side)
      gate_up, down                ExpertStack ([E(+1) * 2I, d] and [E(+1) * d, I])
      shared                       'stacked' (expert #E of the stacks), 'separate' (dense sh_gate_up / sh_down QWeights)
                                   or None
      shared_coef                  'sigmoid' (the reference: sigmoid of the gate logit) or 'one' (always-on, coefficient 1)
    Returns (y [M, d] in x's dtype, dict of intermediates).
    """
    act = act_of(x)
    E, k = L["E"], L["k"]
    lq = (lambda a, w, o=None: linear_q(a, w, o, fast, "orc_fast_linear_q")) if use_fast else linear_q
    lw = (lambda a, w, o=None: linear_w(a, w, o, fast, "orc_fast_linear_w")) if use_fast else linear_w
    r = L["router"]
    logits = lq(x, r, F32) if isinstance(r, QWeight) else lw(x, r, F32)
    if L.get("router_bias") is not None:
        logits[:, :E] += L["router_bias"][None, :]
        logits = np.ascontiguousarray(logits)
    shared, mode = L.get("shared"), L.get("shared_coef", "sigmoid")
    gated = shared is not None and mode == "sigmoid"
    if gated:
        assert logits.shape[1] == E + 1
    ids, coef, err = moe_router(logits, E, k, shared_col=E if (shared == "stacked" and gated) else None, shared_id=E)
    if shared == "stacked" and not gated:
        ids = np.concatenate([ids, np.full((ids.shape[0], 1), E, np.int32)], 1)
        coef = np.concatenate([coef, np.ones((coef.shape[0], 1), np.float32)], 1)
    Estack = E + (1 if shared == "stacked" else 0)
    assert L["gate_up"].E == Estack and L["down"].E == Estack
    h, _ = experts_gather(x, L["gate_up"], ids, swiglu=True, use_fast=use_fast)
    y, _ = experts_combine(h, L["down"], ids, coef, use_fast=use_fast)
    inter = dict(logits=logits, ids=ids, coef=coef, h=h, moe=y.copy())
    if shared == "separate":
        gu = lq(x, L["sh_gate_up"])
        sh = swiglu(gu, L["sh_gate_up"].N // 2)
        sy = lq(sh, L["sh_down"])
        inter["shared_y"] = sy
        if gated:
            moe_shared_add(y, sy, logits, E, E)
        else:
            residual_add(y, sy)
    inter["err"] = err
    return y, inter
