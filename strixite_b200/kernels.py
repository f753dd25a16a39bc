"""Host-side mirror of strixite's kernel interface for the MoE FFN path, over the C ABI of libstrixite_b200.so.

Function names, argument order and meaning follow the reference's C++ declarations (strixite kernels/moe_router.hpp,
moe_grouped.hpp, linear_q4.hpp, linear_q5/6/8.hpp, linear.hpp, swiglu.hpp, residual.hpp, and the dispatchers of
runtime/qweight.hpp); raw device pointers become torch CUDA tensors, `hipStream_t` becomes a torch stream (None = the
current one). torch is used for device memory and streams only - every computation is a kernel of the library.
Failures raise StrixError with the library's message, as the reference throws strix::Error.
"""
import ctypes as C
import enum

import numpy as np
import torch

from ._lib import QMixView, QView, StrixError, call, lib  # noqa: F401


class Act(enum.IntEnum):  # strixite kernels/norm.hpp:20
    F32 = 0
    BF16 = 1


class MoeMath(enum.IntEnum):  # strixite kernels/moe_grouped.hpp:35
    F32 = 0
    WmmaBf16 = 1
    WmmaF16 = 2


kMoeTileRows, kMoeWmmaTileRows, kMoeMaxExperts, kMoeMaxSlots = 16, 64, 1023, 1 << 20  # moe_grouped.hpp:37-40


def act_of(t):
    if t.dtype == torch.float32:
        return Act.F32
    if t.dtype == torch.bfloat16:
        return Act.BF16
    raise StrixError("activations must be float32 or bfloat16, got %s" % t.dtype)


def _dtype(act):
    return torch.float32 if int(act) == Act.F32 else torch.bfloat16


def _p(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise StrixError("expected a CUDA tensor")
    if not t.is_contiguous():
        raise StrixError("expected a contiguous tensor")
    return C.c_void_p(t.data_ptr())


def _s(stream):
    st = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(st.cuda_stream)


def new_err(device="cuda"):
    """>= 3 zeroed uint32 error words (strixite kernels/moe_router.hpp:19-23)."""
    return torch.zeros(4, dtype=torch.int32, device=device)


# ---- weights ---------------------------------------------------------------------------------------------------------


def row_bytes(bits, K):
    return int(lib.strix_row_bytes(bits, K))


class QWeight:
    """A quantized matrix [N, K] on the device with its non-owning view (strixite runtime/q4_device.hpp Q4Device /
    Q4DeviceView and the q5/q6/q8 twins): q uint8 [N * row_bytes], scale / minv int16 (BF16 bits) [N, K / G]."""

    def __init__(self, bits, N, K, G, q, scale, minv):
        self.bits, self.N, self.K, self.G, self.q, self.scale, self.minv = int(bits), int(N), int(K), int(G), q, scale, minv

    def view(self, row0=0, rows=None):
        """strix_qview of rows [row0, row0 + rows) - an expert slice of a stack is a view, never a copy."""
        rows = self.N - row0 if rows is None else rows
        gpr = self.K // self.G
        return QView(self.q.data_ptr() + row0 * row_bytes(self.bits, self.K), self.scale.data_ptr() + row0 * gpr * 2,
                     self.minv.data_ptr() + row0 * gpr * 2, rows, self.K, self.G)

    def nbytes(self):
        return self.q.numel() + 2 * self.scale.numel() + 2 * self.minv.numel()

    @staticmethod
    def upload(bits, N, K, G, q, scale, minv, device="cuda"):
        """From host numpy arrays (uint8, uint16, uint16), checked like Q4Device::upload (check_q4)."""
        call("strix_check_qweight", bits, N, K, G, q.size, scale.size, minv.size)
        tq = torch.from_numpy(np.ascontiguousarray(q)).to(device)
        ts = torch.from_numpy(np.ascontiguousarray(scale).view(np.int16).reshape(N, K // G)).to(device)
        tm = torch.from_numpy(np.ascontiguousarray(minv).view(np.int16).reshape(N, K // G)).to(device)
        return QWeight(bits, N, K, G, tq, ts, tm)

    @staticmethod
    def quantize_host(w, bits, G, device="cuda"):
        """The host quantizer (strixite formats/q4.hpp quantize_q4 ...) on a float32 numpy array [N, K], then upload."""
        q, s, m = quantize(w, bits, G)
        return QWeight.upload(bits, w.shape[0], w.shape[1], G, q, s, m, device)

    @staticmethod
    def quantize_device(w, bits, G, out=None, row0=0, stream=None):
        """The device quantizer on a float32 CUDA tensor [N, K]; bit-identical to the host one. With `out` (a QWeight),
        writes rows [row0, row0 + N) of it instead of allocating."""
        N, K = w.shape
        if out is None:
            out = QWeight.empty(bits, N, K, G, w.device)
            row0 = 0
        err = new_err(w.device)
        v = out.view(row0, N)
        call("strix_quantize_device", bits, _p(w), N, K, G, C.c_void_p(v.q), C.c_void_p(v.scale), C.c_void_p(v.minv), _p(err), _s(stream))
        return out, err

    @staticmethod
    def empty(bits, N, K, G, device="cuda"):
        return QWeight(bits, N, K, G, torch.empty(N * row_bytes(bits, K), dtype=torch.uint8, device=device),
                       torch.empty((N, K // G), dtype=torch.int16, device=device),
                       torch.empty((N, K // G), dtype=torch.int16, device=device))

    def to_host(self):
        return (self.q.cpu().numpy(), self.scale.cpu().numpy().view(np.uint16), self.minv.cpu().numpy().view(np.uint16))


class QMixStack:
    """E experts of N rows each with a format per expert (strix_qmix_view): q holds the experts' code bytes back to
    back (each start 256-byte aligned), bits [E] uint8 and q_off [E] int64 on the device."""

    def __init__(self, E, N, K, G, q, scale, minv, bits, q_off):
        self.E, self.N, self.K, self.G, self.q, self.scale, self.minv, self.bits, self.q_off = E, N, K, G, q, scale, minv, bits, q_off

    def view(self):
        return QMixView(self.q.data_ptr(), self.scale.data_ptr(), self.minv.data_ptr(), self.bits.data_ptr(), self.q_off.data_ptr(),
                        self.E, self.N, self.K, self.G)

    @staticmethod
    def layout(bits_per_expert, N, K):
        """(q_off int64 [E], total bytes) for the given formats."""
        off, total = [], 0
        for b in bits_per_expert:
            off.append(total)
            total += (N * row_bytes(int(b), K) + 255) // 256 * 256
        return np.array(off, np.int64), total

    @staticmethod
    def empty(bits_per_expert, N, K, G, device="cuda"):
        bits_per_expert = np.asarray(bits_per_expert, np.uint8)
        E = len(bits_per_expert)
        off, total = QMixStack.layout(bits_per_expert, N, K)
        return QMixStack(E, N, K, G, torch.zeros(total, dtype=torch.uint8, device=device),
                         torch.empty((E * N, K // G), dtype=torch.int16, device=device),
                         torch.empty((E * N, K // G), dtype=torch.int16, device=device),
                         torch.from_numpy(bits_per_expert).to(device), torch.from_numpy(off).to(device))

    def expert(self, e, bits_host, off_host):
        """A QWeight aliasing expert e's arrays (for filling the stack expert by expert)."""
        b = int(bits_host[e])
        n = self.N * row_bytes(b, self.K)
        return QWeight(b, self.N, self.K, self.G, self.q[int(off_host[e]) : int(off_host[e]) + n], self.scale[e * self.N : (e + 1) * self.N],
                       self.minv[e * self.N : (e + 1) * self.N])

    def nbytes(self):
        return self.q.numel() + 2 * self.scale.numel() + 2 * self.minv.numel()


class QWeightView:
    """strixite runtime/qweight.hpp:23-36 QWeightView: a projection's weight in whichever format it has."""

    def __init__(self, w):
        self.w = w
        self.bits = 0 if isinstance(w, QMixStack) else w.bits

    def N(self):
        return self.w.N

    def K(self):
        return self.w.K


def qweight(w):
    return QWeightView(w)


def quantize(w, bits, G):
    """Host quantizer: float32 numpy [N, K] -> (q uint8, scale uint16 [N, K/G], minv uint16 [N, K/G])."""
    w = np.ascontiguousarray(w, np.float32)
    if w.ndim != 2:
        raise StrixError("quantize: expected a [N, K] array")
    N, K = w.shape
    q = np.zeros(max(N * row_bytes(bits, K), 0), np.uint8)
    s = np.zeros((N, max(K // max(G, 1), 1)), np.uint16)
    m = np.zeros_like(s)
    call("strix_quantize", bits, w.ctypes.data_as(C.c_void_p), N, K, G, q.ctypes.data_as(C.c_void_p), s.ctypes.data_as(C.c_void_p),
         m.ctypes.data_as(C.c_void_p))
    return q, s, m


def dequantize(bits, q, scale, minv, N, K, G):
    out = np.empty((N, K), np.float32)
    call("strix_dequantize", bits, q.ctypes.data_as(C.c_void_p), scale.ctypes.data_as(C.c_void_p), minv.ctypes.data_as(C.c_void_p), N, K, G,
         out.ctypes.data_as(C.c_void_p))
    return out


# ---- router --------------------------------------------------------------------------------------------------------


def moe_router(logits, ld, M, E, k, shared_logit, shared_ld, shared_id, ids, coef, act, err, stream=None):
    """strixite kernels/moe_router.hpp:38-40. shared_logit: None or a tensor whose first element is token 0's gate
    logit (e.g. logits[:, E:] of a merged [M, E + 1] projection)."""
    sp = None if shared_logit is None else C.c_void_p(shared_logit.data_ptr())
    call("strix_moe_router", C.c_void_p(logits.data_ptr()), ld, M, E, k, sp, shared_ld, shared_id, _p(ids), _p(coef), int(act), _p(err), _s(stream))


def check_router_error(err, what):
    call("strix_check_router_error", _p(err), what.encode())


def check_expert_error(err, what):
    call("strix_check_expert_error", _p(err), what.encode())


def moe_shared_add(y, s, gate_logit, gate_ld, M, N, gate_index, act, err, stream=None):
    """strixite kernels/moe_router.hpp:53-54. gate_logit: a float32 tensor whose first element is token 0's logit."""
    call("strix_moe_shared_add", _p(y), _p(s), C.c_void_p(gate_logit.data_ptr()), gate_ld, M, N, gate_index, int(act), _p(err), _s(stream))


def moe_shared_add_inject(y, s, gate_logit, gate_ld, M, N, gate_index, x, w_in, H, act, err, stream=None):
    """strixite kernels/moe_router.hpp:61-63."""
    call("strix_moe_shared_add_inject", _p(y), _p(s), C.c_void_p(gate_logit.data_ptr()), gate_ld, M, N, gate_index, _p(x), _p(w_in), H,
         int(act), _p(err), _s(stream))


# ---- dense projections ---------------------------------------------------------------------------------------------


def _linear_q(bits, x, w, y, M, act, out_act, stream):
    v = w.view() if isinstance(w, QWeight) else w
    call("strix_linear_q%d" % bits, _p(x), C.byref(v), _p(y), M, int(act), int(act if out_act is None else out_act), _s(stream))


def linear_q4(x, w, y, M, act, out_act=None, stream=None):
    """strixite kernels/linear_q4.hpp:26-30."""
    _linear_q(4, x, w, y, M, act, out_act, stream)


def linear_q5(x, w, y, M, act, out_act=None, stream=None):
    """strixite kernels/linear_q5.hpp:14-15."""
    _linear_q(5, x, w, y, M, act, out_act, stream)


def linear_q6(x, w, y, M, act, out_act=None, stream=None):
    """strixite kernels/linear_q6.hpp:14-15."""
    _linear_q(6, x, w, y, M, act, out_act, stream)


def linear_q8(x, w, y, M, act, out_act=None, stream=None):
    """strixite kernels/linear_q8.hpp:13-14."""
    _linear_q(8, x, w, y, M, act, out_act, stream)


def linear_qw(x, w, y, M, act, out_act=None, stream=None):
    """strixite runtime/qweight.hpp:50-61: dispatch on the weight's format."""
    if w.bits not in (4, 5, 6, 8):
        raise StrixError("linear_qw: weight has %d bits (not loaded?), expected 4, 5, 6 or 8" % w.bits)
    _linear_q(w.bits, x, w.w, y, M, act, out_act, stream)


def linear_qw_wmma(x, w, y, M, act, out_act=None, stream=None):
    """strixite runtime/qweight.hpp:63-72 linear_qw_wmma: the dense projection of a quantized matrix on the tensor cores."""
    w = w.w if isinstance(w, QWeightView) else w
    if w.bits not in (4, 5, 6, 8):
        raise StrixError("linear_qw_wmma: weight has %d bits (not loaded?), expected 4, 5, 6 or 8" % w.bits)
    call("strix_linear_q%d_wmma" % w.bits, _p(x), C.byref(w.view()), _p(y), M, int(act), int(act if out_act is None else out_act), _s(stream))


def linear_bf16w_wmma(x, w, y, M, N, K, act, out_act=None, stream=None):
    """strixite kernels/linear_wmma.hpp:27-29."""
    call("strix_linear_bf16w_wmma", _p(x), _p(w), _p(y), M, N, K, int(act), int(act if out_act is None else out_act), _s(stream))


def linear_bf16w(x, w, y, M, N, K, act, out_act=None, stream=None):
    """strixite kernels/linear.hpp:20-26. w: bfloat16 (or int16 bits) [N, K]."""
    call("strix_linear_bf16w", _p(x), _p(w), _p(y), M, N, K, int(act), int(act if out_act is None else out_act), _s(stream))


def linear_f32w(x, w, y, M, N, K, act, out_act=None, stream=None):
    """FP32 weights [N, K] (no reference counterpart: a router kept in FP32)."""
    call("strix_linear_f32w", _p(x), _p(w), _p(y), M, N, K, int(act), int(act if out_act is None else out_act), _s(stream))


# ---- elementwise ---------------------------------------------------------------------------------------------------


def swiglu(gu, h, rows, I, act, stream=None):
    """strixite kernels/swiglu.hpp:21."""
    call("strix_swiglu", _p(gu), _p(h), rows, I, int(act), _s(stream))


def residual_add(x, y, n, act, stream=None):
    """strixite kernels/residual.hpp:17."""
    call("strix_residual_add", _p(x), _p(y), n, int(act), _s(stream))


def hc_inject(x, y, w_in, M, N, H, act, stream=None):
    """strixite kernels/hc.hpp:52-55."""
    call("strix_hc_inject", _p(x), _p(y), _p(w_in), M, N, H, int(act), _s(stream))


# ---- experts, per slot ---------------------------------------------------------------------------------------------


def hc_mix_down(x, w, T, H, d, r, inject, eps, h, w_in, inv, act, stream=None):
    """strixite kernels/hc.hpp:36-39: w a QWeight [r (+ H), H*d] in 4 or 8 bits (folded)."""
    call("strix_hc_mix_down", _p(x), C.byref(w.view()), w.bits, T, H, d, r, int(bool(inject)), float(eps), _p(h), _p(w_in) if inject else None, _p(inv), int(act),
         _s(stream))


def hc_mix_up(h, w_up, x, norm_w, inv, T, H, d, u, act, stream=None):
    """strixite kernels/hc.hpp:47-50: w_up a QWeight [H*d, r] whose arrays are chunk-major (to_chunk_major)."""
    call("strix_hc_mix_up", _p(h), C.byref(w_up.view()), w_up.bits, _p(x), _p(norm_w), _p(inv), T, H, d, _p(u), int(act), _s(stream))


def hc_inject_inv(x, w_in, y, T, H, d, eps, inv, act, stream=None):
    """strixite kernels/hc_wmma.hpp:38-42: hc_inject and the updated streams' inverse RMS in one pass."""
    call("strix_hc_inject_inv", _p(x), _p(w_in), _p(y), T, H, d, float(eps), _p(inv), int(act), _s(stream))


def to_chunk_major(bits, q, scale, minv, N, K, G):
    """strixite formats/q4.hpp:55 on host numpy arrays: (q, scale, minv) re-laid out chunk-major."""
    qo, so, mo = np.empty_like(q), np.empty_like(scale), np.empty_like(minv)
    call("strix_to_chunk_major", bits, q.ctypes.data_as(C.c_void_p), scale.ctypes.data_as(C.c_void_p), minv.ctypes.data_as(C.c_void_p), N, K, G,
         qo.ctypes.data_as(C.c_void_p), so.ctypes.data_as(C.c_void_p), mo.ctypes.data_as(C.c_void_p))
    return qo, so, mo


def _experts(kind, bits, x, w, E, ids, coef, M, A, y, act, err, stream):
    if isinstance(w, QMixStack):
        v = w.view()
        if kind == "combine":
            call("strix_linear_qmix_experts_combine", _p(x), C.byref(v), _p(ids), _p(coef), M, A, _p(y), int(act), _p(err), _s(stream))
        else:
            call("strix_linear_qmix_experts_" + kind, _p(x), C.byref(v), _p(ids), M, A, _p(y), int(act), _p(err), _s(stream))
        return
    v = w.view() if isinstance(w, QWeight) else w
    if kind == "combine":
        call("strix_linear_q%d_experts_combine" % bits, _p(x), C.byref(v), E, _p(ids), _p(coef), M, A, _p(y), int(act), _p(err), _s(stream))
    else:
        call("strix_linear_q%d_experts_%s" % (bits, kind), _p(x), C.byref(v), E, _p(ids), M, A, _p(y), int(act), _p(err), _s(stream))


def linear_q4_experts_gather(x, w, E, ids, M, A, y, act, err, stream=None):
    """strixite kernels/linear_q4.hpp:42-43."""
    _experts("gather", 4, x, w, E, ids, None, M, A, y, act, err, stream)


def linear_q4_experts_combine(h, w, E, ids, coef, M, A, y, act, err, stream=None):
    """strixite kernels/linear_q4.hpp:44-46."""
    _experts("combine", 4, h, w, E, ids, coef, M, A, y, act, err, stream)


def linear_q4_experts_gather_swiglu(x, w, E, ids, M, A, h, act, err, stream=None):
    """strixite kernels/linear_q4.hpp:55-56."""
    _experts("gather_swiglu", 4, x, w, E, ids, None, M, A, h, act, err, stream)


def linear_q5_experts_gather(x, w, E, ids, M, A, y, act, err, stream=None):
    """strixite kernels/linear_q4.hpp:48-49."""
    _experts("gather", 5, x, w, E, ids, None, M, A, y, act, err, stream)


def linear_q5_experts_combine(h, w, E, ids, coef, M, A, y, act, err, stream=None):
    """strixite kernels/linear_q4.hpp:50-52."""
    _experts("combine", 5, h, w, E, ids, coef, M, A, y, act, err, stream)


def linear_q5_experts_gather_swiglu(x, w, E, ids, M, A, h, act, err, stream=None):
    """strixite kernels/linear_q4.hpp:57-58."""
    _experts("gather_swiglu", 5, x, w, E, ids, None, M, A, h, act, err, stream)


def _expert_bits(fn, w):
    if w.bits not in (0, 4, 5):
        raise StrixError("%s: experts have %d bits, expected 4 or 5 (or a per-expert format table)" % (fn, w.bits))
    return w.bits


def linear_qw_experts_gather(x, w, E, ids, M, A, y, act, err, stream=None):
    """strixite runtime/qweight.hpp:75-83 (4 or 5 bits; a QMixStack selects the per-expert-format entry points)."""
    _experts("gather", _expert_bits("linear_qw_experts_gather", w), x, w.w, E, ids, None, M, A, y, act, err, stream)


def linear_qw_experts_gather_swiglu(x, w, E, ids, M, A, h, act, err, stream=None):
    """strixite runtime/qweight.hpp:86-94."""
    _experts("gather_swiglu", _expert_bits("linear_qw_experts_gather_swiglu", w), x, w.w, E, ids, None, M, A, h, act, err, stream)


def linear_qw_experts_combine(h, w, E, ids, coef, M, A, y, act, err, stream=None):
    """strixite runtime/qweight.hpp:95-103."""
    _experts("combine", _expert_bits("linear_qw_experts_combine", w), h, w.w, E, ids, coef, M, A, y, act, err, stream)


# ---- experts, grouped ----------------------------------------------------------------------------------------------


def moe_route_workspace_bytes(M, A, E):
    """strixite kernels/moe_grouped.hpp:43."""
    n = int(lib.strix_moe_route_workspace_bytes(M, A, E))
    if n == 0:
        from ._lib import last_error

        raise StrixError(last_error())
    return n


def moe_group_routes(ids, M, A, E, ws, ws_bytes, err, stream=None):
    """strixite kernels/moe_grouped.hpp:48-49."""
    call("strix_moe_group_routes", _p(ids), M, A, E, _p(ws), ws_bytes, _p(err), _s(stream))


def _gather_grouped(bits, x, w, E, ws, ws_bytes, M, A, y, act, math, stream):
    if isinstance(w, QMixStack):
        call("strix_linear_qmix_experts_gather_grouped", _p(x), C.byref(w.view()), _p(ws), ws_bytes, M, A, _p(y), int(act), int(math), _s(stream))
        return
    v = w.view() if isinstance(w, QWeight) else w
    call("strix_linear_q%d_experts_gather_grouped" % bits, _p(x), C.byref(v), E, _p(ws), ws_bytes, M, A, _p(y), int(act), int(math), _s(stream))


def _combine_grouped(bits, h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, math, stream):
    if isinstance(w, QMixStack):
        call("strix_linear_qmix_experts_combine_grouped", _p(h), C.byref(w.view()), _p(ids), _p(coef), _p(ws), ws_bytes, _p(partial), M, A,
             _p(y), int(act), int(math), _s(stream))
        return
    v = w.view() if isinstance(w, QWeight) else w
    call("strix_linear_q%d_experts_combine_grouped" % bits, _p(h), C.byref(v), E, _p(ids), _p(coef), _p(ws), ws_bytes, _p(partial), M, A,
         _p(y), int(act), int(math), _s(stream))


def linear_q4_experts_gather_grouped(x, w, E, ws, ws_bytes, M, A, y, act, math, stream=None):
    """strixite kernels/moe_grouped.hpp:53-55."""
    _gather_grouped(4, x, w, E, ws, ws_bytes, M, A, y, act, math, stream)


def linear_q5_experts_gather_grouped(x, w, E, ws, ws_bytes, M, A, y, act, math, stream=None):
    """strixite kernels/moe_grouped.hpp:65-67."""
    _gather_grouped(5, x, w, E, ws, ws_bytes, M, A, y, act, math, stream)


def linear_q4_experts_combine_grouped(h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, math, stream=None):
    """strixite kernels/moe_grouped.hpp:60-62."""
    _combine_grouped(4, h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, math, stream)


def moe_combine_reduce(partial, ids, coef, M, A, E, N, y, act, stream=None, pos=None):
    """y[m, :] = sum_a coef[m, a] * partial[m * A + a, :], a ascending, one rounding (the second half of
    strixite kernels/moe_grouped.hpp:60-62 linear_q4_experts_combine_grouped). pos (int64 [M * A]): the row of partial
    that holds each slot, when the rows are not in slot order."""
    call("strix_moe_combine_reduce", _p(partial), None if pos is None else _p(pos), _p(ids), _p(coef), M, A, E, N, _p(y), int(act), _s(stream))


def umma_abort_count():
    """Thread blocks of the tensor-core kernels that abandoned a bounded wait since the library was loaded (0 when healthy)."""
    return int(lib.strix_umma_abort_count())


def workspace_refusal_count():
    """Launches that stored nothing because their grouping workspace was built for other sizes than the call stated."""
    return int(lib.strix_workspace_refusal_count())


def umma_wait_cycles(reset=True):
    """2 x 16 wait-cycle counters of the many-token tensor-core kernels' warp roles (diagnostics)."""
    out = (C.c_ulonglong * 32)()
    lib.strix_umma_wait_cycles(out, 1 if reset else 0)
    return np.array(list(out), dtype=np.uint64).reshape(2, 16)


FIXED_PARTIAL_FLOATS = 1 << 20  # STRIX_FIXED_PARTIAL_FLOATS


def linear_q4_experts_combine_grouped_fixed(h, w, E, ids, coef, ws, ws_bytes, M, A, y, act, math, stream=None):
    """linear_q4_experts_combine_grouped with the partial sums in the library's fixed 4 MiB device array: no buffer to
    pass, nothing allocated; M * A * N <= FIXED_PARTIAL_FLOATS; calls that may overlap in time race on the array."""
    v = w.view() if isinstance(w, QWeight) else w
    call("strix_linear_q4_experts_combine_grouped_fixed", _p(h), C.byref(v), E, _p(ids), _p(coef), _p(ws), ws_bytes, M, A, _p(y), int(act),
         int(math), _s(stream))


def linear_q5_experts_combine_grouped(h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, math, stream=None):
    """strixite kernels/moe_grouped.hpp:68-70."""
    _combine_grouped(5, h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, math, stream)


def linear_qw_experts_gather_grouped(x, w, E, ws, ws_bytes, M, A, y, act, math, stream=None):
    """strixite runtime/qweight.hpp:104-112."""
    _gather_grouped(_expert_bits("linear_qw_experts_gather_grouped", w), x, w.w, E, ws, ws_bytes, M, A, y, act, math, stream)


def linear_qw_experts_combine_grouped(h, w, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, math, stream=None):
    """strixite runtime/qweight.hpp:113-125."""
    _combine_grouped(_expert_bits("linear_qw_experts_combine_grouped", w), h, w.w, E, ids, coef, ws, ws_bytes, partial, M, A, y, act, math,
                     stream)
