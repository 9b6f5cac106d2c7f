"""ctypes binding of include/krasis_b200_seq.h (libkrasis_b200_seq.so) and thin tensor-level wrappers.

The operators work on one step of a serving engine: a flat token axis with per-token and per-sequence int32 tables on the
device (`StepTables`).  All arithmetic runs in the CUDA library; torch owns the buffers.  No fallback: a missing library is an
ImportError that names the build command.
"""
import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_lib", "libkrasis_b200_seq.so")

_P, _I, _L, _F = C.c_void_p, C.c_int, C.c_longlong, C.c_float
SIGNATURES = {
    "kb2_seq_last_error": (C.c_char_p, []),
    "kb2_seq_total_launches": (C.c_longlong, []),
    "kb2_seq_embed": (_I, [_P, _I, _P, _P, _I, _I, _F, _P]),
    "kb2_seq_gemm": (_I, [_P, _I, _L, _P, _I, _L, _P, _I, _L, _I, _I, _I, _I, _L, _L, _L, _P]),
    "kb2_seq_residual_norm": (_I, [_P, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _P]),
    "kb2_seq_act_mul": (_I, [_P, _I, _P, _I, _I, _I, _P]),
    "kb2_seq_side_gate": (_I, [_P, _P, _I, _L, _P, _I, _I, _I, _P, _I, _P]),
    "kb2_seq_latent_prep": (_I, [_P, _L, _I, _I, _I, _I, _I, _P, _F, _P, _I, _F, _P, _P, _P, _I, _I, _P, _P, _I, _P, _L, _P]),
    "kb2_seq_latent_window_attn": (_I, [_P, _P, _L, _I, _I, _I, _I, _I, _P, _P, _I, _P, _P, _P, _I, _I, _P, _F, _I, _P, _P, _I, _I, _P, _P, _P]),
    "kb2_seq_conv_silu": (_I, [_P, _L, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P]),
    "kb2_seq_delta_rule": (_I, [_P, _I, _P, _L, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _F, _P, _P, _P, _P, _P, _I, _P]),
    "kb2_seq_conv": (_I, [_P, _L, _I, _I, _I, _I, _P, _P, _I, _P, _P, _P, _P, _P, _P]),
    "kb2_seq_residual_scale_rms": (_I, [_P, _P, _F, _P, _F, _P, _I, _I, _I, _F, _P]),
    "kb2_seq_delta_rule_ch": (_I, [_P, _I, _P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _F, _P, _P, _P, _P, _P, _I, _P]),
    "kb2_seq_residual_add_norm": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _P]),
    "kb2_seq_head_kv_prep": (_I, [_P, _L, _I, _I, _I, _I, _I, _I, _P, _P, _P, _F, _P, _I, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _P, _P]),
    "kb2_seq_kv_pool": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _I, _I, _P]),
    "kb2_seq_paged_attn": (_I, [_P, _L, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _P, _P, _I, _I, _F, _I, _I, _P, _I, _P, _P, _P, _I, _F, _P, _I,
                                _P, _P, _I, _P]),
    "kb2_seq_pool_merge": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _P, _I, _P]),
    "kb2_seq_attn_finish": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _F, _F, _P, _L, _P, _I, _P, _P, _I, _I, _P, _P, _I, _P]),
    "kb2_seq_glu": (_I, [_P, _I, _L, _P, _I, _L, _I, _I, _F, _F, _P, _I, _P]),
    "kb2_seq_route": (_I, [_P, _L, _I, _I, _P, _I, _I, _I, _I, _I, _F, _P, _P, _I, _P]),
    "kb2_seq_moe_tile_rows": (_I, []),
    "kb2_seq_moe_bin": (_I, [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P, _L, _P, _P]),
    "kb2_seq_moe_gemm": (_I, [_P, _I, _L, _P, _I, _P, _I, _L, _L, _P, _I, _L, _I, _I, _P, _P, _I, _I, _P]),
    "kb2_seq_moe_gemv": (_I, [_P, _I, _L, _I, _P, _I, _P, _I, _L, _L, _P, _I, _L, _I, _I, _I, _P]),
    "kb2_seq_moe_combine": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _P, _P, _I, _P, _L, _P]),
    "kb2_seq_gla": (_I, [_P, _L, _I, _I, _I, _P, _L, _P, _F, _F, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "kb2_seq_selective_scan": (_I, [_P, _L, _P, _L, _P, _P, _L, _I, _P, _L, _I, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _I, _P]),
    "kb2_seq_head_norm_gate": (_I, [_P, _L, _P, _F, _P, _L, _I, _I, _I, _I, _P, _I, _P]),
    "kb2_seq_rms_rows": (_I, [_P, _L, _I, _P, _F, _P, _I, _L, _I, _P]),
    "kb2_seq_branch_merge": (_I, [_P, _P, _P, _P, _F, _F, _P, _I, _I, _P]),
    "kb2_seq_depth_mix": (_I, [_P, _L, _I, _P, _P, _P, _P, _P, _I, _I, _I, _F, _P]),
}

_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m krasis_b200.build --seq-only` "
                              "(krasis_b200 has no CPU or PyTorch fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class SeqOpsError(RuntimeError):
    pass


def check(rc: int):
    if rc == 0:
        return
    msg = load().kb2_seq_last_error().decode()
    if rc == 2:
        raise ValueError(msg)
    raise SeqOpsError(msg)


def total_launches() -> int:
    return int(load().kb2_seq_total_launches())


def dt_code(dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise ValueError(f"unsupported dtype {dtype}: float32 or bfloat16")


def _s(t) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _cuda(t, name):
    if not t.is_cuda:
        raise ValueError(f"{name}: expected a CUDA tensor (krasis_b200 has no CPU path)")


def _ptr(t):
    return t.data_ptr() if t is not None else None


class StepTables:
    """The int32 tables of one step, packed into one pinned host buffer and copied to the device in one transfer.

    entries: [(tokens, start_position, state_slot, page_list)] in batch order."""

    def __init__(self, entries, device, pad_pages_to: int = 1, device_buf=None):
        """pad_pages_to rounds the page-list width up (fewer distinct shapes); device_buf, if given, is a device int32 buffer of the
        right size that receives the tables (a captured CUDA graph reads its tables from a fixed buffer)."""
        import numpy as np
        S = len(entries)
        T = sum(len(e[0]) for e in entries)
        maxp = max(1, max(len(e[3]) for e in entries))
        maxp = (maxp + pad_pages_to - 1) // pad_pages_to * pad_pages_to
        n = 3 * T + (S + 1) + S + S * maxp
        host = torch.empty(n, dtype=torch.int32, pin_memory=torch.cuda.is_available())
        a = host.numpy()
        cu = 0
        o_pos, o_seq, o_cu, o_slot, o_pg = T, 2 * T, 3 * T, 3 * T + S + 1, 3 * T + 2 * S + 1
        a[o_pg:] = 0
        for s, (toks, start, slot, pages) in enumerate(entries):
            k = len(toks)
            a[cu:cu + k] = np.asarray(toks, dtype=np.int32)
            a[o_pos + cu:o_pos + cu + k] = np.arange(start, start + k, dtype=np.int32)
            a[o_seq + cu:o_seq + cu + k] = s
            a[o_cu + s] = cu
            a[o_slot + s] = slot
            a[o_pg + s * maxp:o_pg + s * maxp + len(pages)] = np.asarray(pages, dtype=np.int32)
            cu += k
        a[o_cu + S] = cu
        self.T, self.S, self.max_pages = T, S, maxp
        # host copy of the step's layout: (first row, tokens, first position, page list) per sequence
        self.layout, row = [], 0
        for toks, start, _, pages in entries:
            self.layout.append((row, len(toks), int(start), list(pages)))
            row += len(toks)
        self._key_rows = {}
        self.max_portion = max(len(e[0]) for e in entries)
        if device_buf is not None:
            if device_buf.numel() != n:
                raise ValueError("device_buf does not fit this step's tables")
            device_buf.copy_(host, non_blocking=True)
            self.buf = device_buf
        else:
            self.buf = host.to(device, non_blocking=True)
        self.numel = n
        self._host = host
        self.tokens, self.positions, self.seq_of = self.buf[:T], self.buf[o_pos:o_pos + T], self.buf[o_seq:o_seq + T]
        self.cu, self.slots, self.pages = self.buf[o_cu:o_cu + S + 1], self.buf[o_slot:o_slot + S], self.buf[o_pg:]
        self.h2d_bytes = n * 4


def key_rows(tb: StepTables, s: int, window: int, page_size: int):
    """Cache rows of the keys sequence s needs in this step under a sliding window: (first key position, int64 rows on the device),
    computed once per step and window size."""
    key = (s, window, page_size)
    if key not in tb._key_rows:
        import numpy as np
        _, n, start, pages = tb.layout[s]
        lo = max(0, start - window + 1)
        j = np.arange(lo, start + n, dtype=np.int64)
        rows = np.asarray(pages, dtype=np.int64)[j // page_size] * page_size + j % page_size
        tb._key_rows[key] = (lo, torch.from_numpy(rows).to(tb.buf.device, non_blocking=True))
    return tb._key_rows[key]


def embed(table: torch.Tensor, tokens: torch.Tensor, scale: float) -> torch.Tensor:
    _cuda(table, "table")
    T, W = tokens.shape[0], table.shape[1]
    x = torch.empty((T, W), dtype=torch.float32, device=table.device)
    check(load().kb2_seq_embed(table.data_ptr(), dt_code(table.dtype), tokens.data_ptr(), x.data_ptr(), T, W, float(scale), _s(table)))
    return x


def gemm(a: torch.Tensor, w: torch.Tensor, out_dtype=torch.float32, out: torch.Tensor = None) -> torch.Tensor:
    """a [M, K] (row stride free) times w [N, K]^T -> [M, N]."""
    _cuda(a, "a")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or a.stride(1) != 1 or w.stride(1) != 1:
        raise ValueError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    check(load().kb2_seq_gemm(a.data_ptr(), dt_code(a.dtype), a.stride(0), w.data_ptr(), dt_code(w.dtype), w.stride(0), out.data_ptr(),
                              dt_code(out.dtype), out.stride(0), M, N, K, 1, 0, 0, 0, _s(a)))
    return out


def gemm_heads(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Per-head product: a [M, H, K] (any strides with unit last stride), w [H, N, K] -> out [M, H, N]."""
    M, H, K = a.shape
    N = w.shape[1]
    if w.shape[0] != H or w.shape[2] != K or out.shape != (M, H, N) or a.stride(2) != 1 or out.stride(2) != 1 or not w.is_contiguous():
        raise ValueError("gemm_heads: shape mismatch")
    check(load().kb2_seq_gemm(a.data_ptr(), dt_code(a.dtype), a.stride(0), w.data_ptr(), dt_code(w.dtype), K, out.data_ptr(),
                              dt_code(out.dtype), out.stride(0), M, N, K, H, a.stride(1), N * K, out.stride(1), _s(a)))
    return out


def residual_norm(x, y=None, y_norm=None, x0=None, out_norm=None, out_dtype=torch.float32, eps=1e-5):
    """x (fp32, in place) += norm(y) [+ x0]; returns layer_norm(x) with out_norm = (weight, bias) or None.
    y_norm = ("layer", w, b) | ("rms", w)."""
    T, W = x.shape
    mode, wa, ba = 0, None, None
    if y is not None:
        mode = 1 if y_norm[0] == "layer" else 2
        wa, ba = y_norm[1], (y_norm[2] if mode == 1 else None)
        if y.dtype != torch.float32 or not y.is_contiguous():
            raise ValueError("residual_norm: y must be contiguous fp32")
    h = torch.empty((T, W), dtype=out_dtype, device=x.device) if out_norm is not None else None
    wb, bb = out_norm if out_norm is not None else (None, None)
    check(load().kb2_seq_residual_norm(x.data_ptr(), _ptr(y), mode, _ptr(wa), _ptr(ba), _ptr(x0), _ptr(wb), _ptr(bb), _ptr(h),
                                       dt_code(out_dtype), T, W, float(eps), _s(x)))
    return h


def act_mul(gate_up: torch.Tensor, out_dtype) -> torch.Tensor:
    T, F2 = gate_up.shape
    out = torch.empty((T, F2 // 2), dtype=out_dtype, device=gate_up.device)
    check(load().kb2_seq_act_mul(gate_up.data_ptr(), dt_code(gate_up.dtype), out.data_ptr(), dt_code(out_dtype), T, F2 // 2, _s(gate_up)))
    return out


def side_gate(g: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, col0: int, out_dtype) -> torch.Tensor:
    T, dim = g.shape
    out = torch.empty((T, dim), dtype=out_dtype, device=g.device)
    check(load().kb2_seq_side_gate(g.data_ptr(), table.data_ptr(), dt_code(table.dtype), table.stride(0), tokens.data_ptr(), col0, dim, T,
                                   out.data_ptr(), dt_code(out_dtype), _s(g)))
    return out


def residual_add_norm(x, y=None, y2=None, out_norm=None, out_dtype=torch.float32, eps=1e-5):
    """x (fp32, in place) += (y + y2); returns layer_norm(x) with out_norm = (weight, bias or None), or None."""
    T, W = x.shape
    for t in (y, y2):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.shape != x.shape):
            raise ValueError("residual_add_norm: addends must be contiguous fp32 of x's shape")
    h = torch.empty((T, W), dtype=out_dtype, device=x.device) if out_norm is not None else None
    wb, bb = out_norm if out_norm is not None else (None, None)
    check(load().kb2_seq_residual_add_norm(x.data_ptr(), _ptr(y), _ptr(y2), _ptr(wb), _ptr(bb), _ptr(h), dt_code(out_dtype), T, W, float(eps),
                                           _s(x)))
    return h


GLU_GELU_TANH, GLU_SILU, GLU_CLAMPED_SWISH, ACT_RELU2 = 0, 1, 2, 3


def glu(gate_up: torch.Tensor, out_dtype, kind: int, limit: float = 0.0, alpha: float = 1.0, n_tiles=None, tile_rows: int = 0) -> torch.Tensor:
    """[rows, 2F] = [gate | up] -> [rows, F]; ACT_RELU2: [rows, F] -> relu(.)^2 of it, no up half.  See kb2_seq_glu for the kinds."""
    rows, F2 = gate_up.shape
    F = F2 if kind == ACT_RELU2 else F2 // 2
    out = torch.empty((rows, F), dtype=out_dtype, device=gate_up.device)
    check(load().kb2_seq_glu(gate_up.data_ptr(), dt_code(gate_up.dtype), gate_up.stride(0), out.data_ptr(), dt_code(out_dtype), rows, F,
                             int(kind), float(limit), float(alpha), _ptr(n_tiles), int(tile_rows), _s(gate_up)))
    return out


def residual_scale_rms(x, y=None, y_mult: float = 1.0, norm=None, w_shift: float = 0.0, out_dtype=torch.float32, eps=1e-5, in_place=False):
    """x (fp32, in place) += y_mult * y; returns x / rms(x) * (w_shift + norm) in out_dtype (None without `norm`).
    in_place: the normed row replaces x itself (fp32, no addend)."""
    T, W = x.shape
    if y is not None and (y.dtype != torch.float32 or not y.is_contiguous() or y.shape != x.shape):
        raise ValueError("residual_scale_rms: the addend must be contiguous fp32 of x's shape")
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise ValueError("residual_scale_rms: x must be contiguous fp32")
    h = None
    if norm is not None:
        h = x if in_place else torch.empty((T, W), dtype=out_dtype, device=x.device)
    check(load().kb2_seq_residual_scale_rms(x.data_ptr(), _ptr(y), float(y_mult), _ptr(norm), float(w_shift), _ptr(h),
                                            dt_code(h.dtype) if h is not None else 0, T, W, float(eps), _s(x)))
    return h


def conv(proj: torch.Tensor, C: int, taps: torch.Tensor, bias, act: bool, tail: torch.Tensor, tb: "StepTables", bias_after: bool = False) -> torch.Tensor:
    """Short causal convolution over time on the first C columns of proj [T, >= C] fp32 (+ bias), with the carried tail
    [slots, C, taps - 1] read and advanced; silu on the result if act.  bias_after: the bias is added to the convolution's result
    (ahead of the activation) instead of to its inputs."""
    T, K = proj.shape[0], taps.shape[1]
    out = torch.empty((T, C), dtype=torch.float32, device=proj.device)
    check(load().kb2_seq_conv(proj.data_ptr(), proj.stride(0), T, tb.S, C, K, taps.data_ptr(), _ptr(bias), int(bool(act)) + 2 * int(bool(bias_after)), tail.data_ptr(),
                              tb.seq_of.data_ptr(), tb.cu.data_ptr(), tb.slots.data_ptr(), out.data_ptr(), _s(proj)))
    return out


def route(z: torch.Tensor, correction, top: int, groups: int = 1, keep: int = 1, score: str = "softmax", renorm: bool = False,
          out_scale: float = 1.0, group_score: str = "max", experts: int = None):
    """Router logits z [T, >= E] fp32 -> (ids [T, top] int32, weights [T, top] fp32).  experts: E when z carries further columns.
    group_score: "max" (a group's largest choice) or "top2" (the sum of its two largest)."""
    if z.dtype != torch.float32 or z.stride(1) != 1:
        raise ValueError("route: logits must be fp32 rows")
    T, E = z.shape
    E = E if experts is None else int(experts)
    ids = torch.empty((T, top), dtype=torch.int32, device=z.device)
    w = torch.empty((T, top), dtype=torch.float32, device=z.device)
    check(load().kb2_seq_route(z.data_ptr(), z.stride(0), T, E, _ptr(correction), {"softmax": 0, "sigmoid": 1}[score], int(groups), int(keep),
                               int(top), int(renorm), float(out_scale), ids.data_ptr(), w.data_ptr(), {"max": 0, "top2": 1}[group_score],
                               _s(z)))
    return ids, w


def rms_rows(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype) -> torch.Tensor:
    """x [T, n] fp32 rows (row stride free) -> x / rms(x) * w, contiguous in out_dtype."""
    T, n = x.shape
    if x.dtype != torch.float32 or x.stride(1) != 1:
        raise ValueError("rms_rows: fp32 rows")
    out = torch.empty((T, n), dtype=out_dtype, device=x.device)
    check(load().kb2_seq_rms_rows(x.data_ptr(), x.stride(0), n, w.data_ptr(), float(eps), out.data_ptr(), dt_code(out_dtype), n, T, _s(x)))
    return out


def head_norm_gate(o: torch.Tensor, H: int, dv: int, out_dtype, norm=None, eps: float = 0.0, gate=None, gate_act: str = "silu") -> torch.Tensor:
    """o [T, >= H dv] fp32 -> per head o / rms(o) * norm (if norm) times silu | sigmoid of gate [T, >= H dv] (if gate), in out_dtype."""
    T = o.shape[0]
    out = torch.empty((T, H * dv), dtype=out_dtype, device=o.device)
    check(load().kb2_seq_head_norm_gate(o.data_ptr(), o.stride(0), _ptr(norm), float(eps), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                        {"silu": 0, "sigmoid": 1}[gate_act], T, H, dv, out.data_ptr(), dt_code(out_dtype), _s(o)))
    return out


def branch_merge(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float, coef: float = 0.5) -> torch.Tensor:
    """coef (a / rms(a) * wa + b / rms(b) * wb) per row; a, b contiguous fp32 [T, W]."""
    for t in (a, b):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.shape != a.shape:
            raise ValueError("branch_merge: contiguous fp32 rows of one shape")
    out = torch.empty_like(a)
    check(load().kb2_seq_branch_merge(a.data_ptr(), b.data_ptr(), wa.data_ptr(), wb.data_ptr(), float(eps), float(coef), out.data_ptr(),
                                      a.shape[0], a.shape[1], _s(a)))
    return out


def depth_mix(stack: torch.Tensor, n: int, coef: torch.Tensor, x: torch.Tensor, y=None, norm=None, out_dtype=torch.float32, eps: float = 1e-5):
    """stack [>= n, T, W] fp32 holds n - 1 earlier results; entry n - 1 <- x + y; x <- sum_j coef[j] stack[j]; returns
    x / rms(x) * norm in out_dtype (None without `norm`)."""
    T, W = x.shape
    if stack.dtype != torch.float32 or not stack.is_contiguous() or stack.shape[0] < n or stack.shape[1:] != x.shape or coef.numel() < n:
        raise ValueError("depth_mix: stack [>= n, T, W] fp32 and n coefficients")
    if x.dtype != torch.float32 or not x.is_contiguous() or (y is not None and (y.dtype != torch.float32 or not y.is_contiguous())):
        raise ValueError("depth_mix: x and y must be contiguous fp32")
    h = torch.empty((T, W), dtype=out_dtype, device=x.device) if norm is not None else None
    check(load().kb2_seq_depth_mix(stack.data_ptr(), stack.stride(0), n, coef.data_ptr(), x.data_ptr(), _ptr(y), _ptr(norm), _ptr(h),
                                   dt_code(out_dtype) if h is not None else 0, T, W, float(eps), _s(x)))
    return h
