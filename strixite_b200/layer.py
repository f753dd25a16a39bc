"""The MoE sublayer object (strix_moe_layer_* of the C ABI): strixite's per-layer driver, runtime/qwen4exp.cpp:1126-1186,
with its session buffers. Weights stay with the caller (torch tensors inside QWeight / QMixStack); the layer owns only
workspaces, created once for `max_tokens`."""
import ctypes as C

import numpy as np
import torch

from . import kernels as K
from ._lib import QMixView, QView, StrixError, call, lib

SHARED_NONE, SHARED_STACKED, SHARED_SEPARATE = 0, 1, 2
COEF_SIGMOID, COEF_ONE = 0, 1
ROUTER_F32, ROUTER_BF16, ROUTER_Q = 0, 1, 2
kGroupedMinTokens = 6  # strixite runtime/qwen4exp.hpp:266


class _Desc(C.Structure):
    _fields_ = [
        ("d", C.c_int64), ("I", C.c_int64), ("E", C.c_int64), ("k", C.c_int64),
        ("act", C.c_int), ("shared_mode", C.c_int), ("shared_coef_mode", C.c_int), ("router_kind", C.c_int),
        ("router_w", C.c_void_p), ("router_bits", C.c_int), ("router_q", QView), ("router_bias", C.c_void_p),
        ("experts_mixed", C.c_int), ("gate_up_bits", C.c_int), ("down_bits", C.c_int),
        ("gate_up", QView), ("down", QView), ("gate_up_mix", QMixView), ("down_mix", QMixView),
        ("sh_gate_up_bits", C.c_int), ("sh_down_bits", C.c_int), ("sh_gate_up", QView), ("sh_down", QView),
        ("max_tokens", C.c_int64), ("grouped_min_tokens", C.c_int64), ("math", C.c_int), ("tensor_min_tokens", C.c_int64), ("decode_impl", C.c_int),
    ]


lib.strix_moe_layer_create.argtypes = [C.POINTER(_Desc), C.POINTER(C.c_void_p)]
lib.strix_moe_layer_create.restype = C.c_int
lib.strix_moe_layer_destroy.argtypes = [C.c_void_p]
lib.strix_moe_layer_destroy.restype = None
lib.strix_moe_layer_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
lib.strix_moe_layer_forward.restype = C.c_int
lib.strix_moe_layer_forward_host.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
lib.strix_moe_layer_forward_host.restype = C.c_int
lib.strix_moe_stack_forward.argtypes = [C.POINTER(C.c_void_p), C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
lib.strix_moe_stack_forward.restype = C.c_int
lib.strix_moe_layer_probe.argtypes = [C.c_void_p, C.c_char_p]
lib.strix_moe_layer_probe.restype = C.c_void_p
lib.strix_moe_layer_reset_errors.argtypes = [C.c_void_p, C.c_void_p]
lib.strix_moe_layer_reset_errors.restype = C.c_int
lib.strix_moe_layer_experts_partial.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_void_p]
lib.strix_moe_layer_experts_partial.restype = C.c_int


class MoeLayer:
    """One MoE FFN sublayer.

    router: float32 / bfloat16 tensor [R, d] or a QWeight [R, d]; R = E + 1 when the shared expert is gated
            (shared_coef='sigmoid', the reference: row E is its gate), else E.
    gate_up, down: QWeight stacks ([Estack*2I, d], [Estack*d, I]; 4 or 5 bits) or QMixStack (a format per expert).
    shared: None | 'stacked' (expert #E of the stacks) | 'separate' (sh_gate_up / sh_down QWeights).
    """

    def __init__(self, d, I, E, k, act, router, gate_up, down, shared=None, shared_coef="sigmoid", sh_gate_up=None, sh_down=None,
                 router_bias=None, max_tokens=8, grouped_min_tokens=kGroupedMinTokens, math=K.MoeMath.F32, decode_impl=0, tensor_min_tokens=0):
        self._keep = [router, gate_up, down, sh_gate_up, sh_down, router_bias]  # the views must outlive the layer
        self.d, self.I, self.E, self.k, self.act, self.max_tokens = d, I, E, k, K.Act(act), max_tokens
        self.A = k + (1 if shared == "stacked" else 0)
        ds = _Desc()
        ds.d, ds.I, ds.E, ds.k, ds.act = d, I, E, k, int(act)
        ds.shared_mode = {None: SHARED_NONE, "stacked": SHARED_STACKED, "separate": SHARED_SEPARATE}[shared]
        ds.shared_coef_mode = {"sigmoid": COEF_SIGMOID, "one": COEF_ONE}[shared_coef]
        self.gated = shared is not None and shared_coef == "sigmoid"
        self.router_rows = E + (1 if self.gated else 0)
        if isinstance(router, K.QWeight):
            ds.router_kind, ds.router_bits, ds.router_q = ROUTER_Q, router.bits, router.view()
        else:
            if tuple(router.shape) != (self.router_rows, d):
                raise StrixError("MoeLayer: router must be [%d, %d], got %s" % (self.router_rows, d, tuple(router.shape)))
            ds.router_kind = ROUTER_F32 if router.dtype == torch.float32 else ROUTER_BF16
            ds.router_w = router.data_ptr()
        if router_bias is not None:
            ds.router_bias = router_bias.data_ptr()
        if isinstance(gate_up, K.QMixStack):
            ds.experts_mixed, ds.gate_up_mix, ds.down_mix = 1, gate_up.view(), down.view()
        else:
            ds.gate_up_bits, ds.down_bits, ds.gate_up, ds.down = gate_up.bits, down.bits, gate_up.view(), down.view()
        if shared == "separate":
            ds.sh_gate_up_bits, ds.sh_down_bits, ds.sh_gate_up, ds.sh_down = sh_gate_up.bits, sh_down.bits, sh_gate_up.view(), sh_down.view()
        ds.max_tokens, ds.grouped_min_tokens, ds.math, ds.decode_impl = max_tokens, grouped_min_tokens, int(math), int(decode_impl)
        ds.tensor_min_tokens = int(tensor_min_tokens)
        self._desc = ds
        h = C.c_void_p()
        call("strix_moe_layer_create", C.byref(ds), C.byref(h))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            lib.strix_moe_layer_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def forward(self, x, y=None, stream=None):
        """y[M, d] = MoE(x[M, d]) on the device."""
        M = x.shape[0]
        y = torch.empty_like(x) if y is None else y
        call("strix_moe_layer_forward", self._h, K._p(x), M, K._p(y), K._s(stream))
        return y

    def forward_host(self, x_host, y_host=None, stream=None):
        """The same through host numpy buffers (float32, or uint16 BF16 bits): copies in, runs, copies back, one sync."""
        M = x_host.shape[0]
        y_host = np.empty_like(x_host) if y_host is None else y_host
        call("strix_moe_layer_forward_host", self._h, x_host.ctypes.data_as(C.c_void_p), M, y_host.ctypes.data_as(C.c_void_p), K._s(stream))
        return y_host

    def experts_partial(self, rows, ids, partial=None, stream=None, row_index=None):
        """partial[i, :] = W_down[ids[i]] * SwiGLU(W_gate_up[ids[i]] * row_i) for a batch of routed slots: the expert half of an
        expert-parallel layer, FP32 or (a float16 `partial` tensor) F16. row_i = rows[row_index[i]] (int32 index), or rows[i]
        when row_index is None."""
        n = ids.shape[0]
        partial = torch.empty((n, self.d), dtype=torch.float32, device=rows.device) if partial is None else partial
        if partial.dtype not in (torch.float32, torch.float16):
            raise StrixError("experts_partial: partial must be float32 or float16, got %s" % partial.dtype)
        call("strix_moe_layer_experts_partial", self._h, K._p(rows), None if row_index is None else K._p(row_index), K._p(ids), n, K._p(partial),
             1 if partial.dtype == torch.float16 else 0, K._s(stream))
        return partial

    @property
    def streams_decode(self):
        """True when forwards of at most 8 tokens run the single streaming decode kernel (its shapes and formats fit);
        False when they run the per-function kernels in the reference's sequence."""
        return bool(lib.strix_moe_layer_probe(self._h, b"decode_sync"))

    def reset_errors(self, stream=None):
        call("strix_moe_layer_reset_errors", self._h, K._s(stream))

    def probe(self, name, M):
        """A copy of a named intermediate of the last forward (the reference's probes, runtime/qwen4exp.hpp:179-188)."""
        p = lib.strix_moe_layer_probe(self._h, name.encode())
        if not p:
            raise StrixError("MoeLayer.probe: unknown buffer %r" % name)
        shapes = {
            "router_logits": ((M, self.router_rows), torch.float32), "router_ids": ((M, self.A), torch.int32),
            "router_coef": ((M, self.A), torch.float32), "experts_h": ((M, self.A, self.I), K._dtype(self.act)),
            "shared_h": ((M, self.I), K._dtype(self.act)), "shared_y": ((M, self.d), K._dtype(self.act)), "err": ((6,), torch.int32), "decode_sync": ((128,), torch.int32),
        }
        bf16 = shapes[name][1] == torch.bfloat16
        shape, dt = shapes[name]
        torch.cuda.current_stream().synchronize()
        out = torch.as_tensor(_DevArray(p, shape, dt), device="cuda").clone()
        return out.view(torch.bfloat16) if bf16 else out


class _DevArray:
    """A device buffer of the library seen through __cuda_array_interface__ (read by torch.as_tensor, then cloned)."""

    _TYPESTR = {torch.float32: "<f4", torch.int32: "<i4", torch.bfloat16: "<i2"}

    def __init__(self, ptr, shape, dtype):
        self._bf16 = dtype == torch.bfloat16
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": self._TYPESTR[dtype], "data": (int(ptr), False), "version": 3}


def stack_forward(layers, x, tmp=None, stream=None):
    """x[M, d] += MoE_l(x) for each layer in order (strix_moe_stack_forward)."""
    tmp = torch.empty_like(x) if tmp is None else tmp
    arr = (C.c_void_p * len(layers))(*[l._h for l in layers])
    call("strix_moe_stack_forward", arr, len(layers), K._p(x), x.shape[0], K._p(tmp), K._s(stream))
    return x
