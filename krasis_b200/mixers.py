"""Token mixers and sublayers for ragged-batch serving (prefill portions and decoded tokens in one step).

Each class owns its weights on the device, takes its constants as constructor arguments and runs on the kernels of
libkrasis_b200_seq (`krasis_b200.seqops`): a model composes them (krasis_b200/vofelix.py).

  WindowLatentAttention   attention over a cached low-rank latent with one shared rotated key part, interleaved rotary positions
                          with YaRN frequency blending, a sliding window and a per-head softmax sink (optional: queries through a
                          normed latent of their own, no sink, a sigmoid output gate per element)
  GatedDeltaMixer         short causal convolutions on q / k / v, unit-norm q and k, gated delta-rule state per head in fp32
                          slots, per-head RMS norm of the read-out with a SiLU gate
  MultiMapAttention       grouped-query attention over a per-head paged cache whose heads carry several attention maps (keys per
                          map, shared values) combined with fixed coefficients (differential attention: a1 - lambda a2), with
                          query / key RMS norm, interleaved rotary positions on part of the dimensions with linear scaling, a causal
                          mask cut into chunks and / or a sliding window, a unit norm per head, a per-head sigmoid output gate, and
                          optionally another layer's cached keys and values instead of projections of its own
                          (further options: a short causal convolution on q / k / v after the projection, one RMS norm over the whole
                          of q and of k, rotation of dimension i with i + dims / 2, a frequency table of the caller, tanh soft-capped
                          scores, a softmax sink per head, mean-pooled blocks of keys and values before the window, values cached
                          rotated by their positions with the output turned back, an output gate per element)
  GatedLinearAttention    S <- diag(alpha) S + k v^T with one decay per key channel, alpha = sigmoid(.)^(1 / tau) from a low-rank
                          projection; per-head RMS norm of the read-out with a SiLU gate
  SelectiveScan           Mamba: input / gate projection, short causal convolution, input-dependent step sizes and B / C, diagonal
                          state per channel in fp32 slots
  SideBySide              two mixers that read the same input: each output RMS-normed over the width, then averaged
  ChannelDeltaMixer       the gated delta rule with one decay per head and key channel (low-rank decay and output-gate projections,
                          sigmoid output gate)
  GatedMLP                down(act(gate h) * (up h)): tanh-GELU, SiLU, or the clamped swish form g' sigmoid(a g') (u' + 1); without a
                          gate: down(relu(up h)^2)
  RoutedExperts           softmax / sigmoid router with a choice correction, expert groups (scored by their best or their two best
                          outputs) and identity experts, top-k experts of either form (binned tile GEMMs; a GEMV form for steps of few
                          tokens) plus an optional shared expert with an optional per-token sigmoid gate
  TokenSideInput          per-layer token table slice, gated by a projection of the residual stream, RMS-normed
`lin(a, w, out_dtype)` picks the GEMM: the tcgen05 kernel of the core library for large aligned bf16 products, the generic
kernel of the sequence library otherwise (any shape, fp32 or bf16).
"""
import math
import os

import torch

from . import seqops as ops


_core = None


def _core_lib():
    """The core library's tcgen05 GEMM, if that library has been built (it is optional for models that run on seqops alone)."""
    global _core
    if _core is None:
        _core = False
        if os.environ.get("KB2_SEQ_TCGEN05", "1") != "0":
            try:
                from . import capi
                if os.path.exists(capi.LIB_PATH):
                    _core = capi.load()
            except Exception:       # noqa: BLE001 — optional accelerator; the generic kernel computes the same product
                _core = False
    return _core


def lin(a: torch.Tensor, w: torch.Tensor, out_dtype=torch.float32, min_n: int = 256) -> torch.Tensor:
    """a [M, K] @ w [N, K]^T with fp32 accumulation.  min_n: the narrowest output that still goes to the tcgen05 kernel (its tiles are
    256 columns wide; a router's few columns are worth it all the same when the step is long)."""
    M, K = a.shape
    N = w.shape[0]
    if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M >= 256 and K % 64 == 0 and N % 16 == 0 and N >= min_n
            and a.is_contiguous() and w.is_contiguous()):
        core = _core_lib()
        if core:
            from . import capi
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
            capi.check(core.kb2_linear_bf16(a.data_ptr(), w.data_ptr(), None, out.data_ptr(), M, N, K, int(out_dtype == torch.float32),
                                            a.device.index or 0, torch.cuda.current_stream(a.device).cuda_stream))
            return out
    return ops.gemm(a, w, out_dtype)


def yarn_table(dims: int, base: float, scaling):
    """Angular frequency of each rotated pair (fp64) and the amplitude both sin and cos carry.
    scaling = {factor, original, fast, slow} or None: pairs that turn more than `fast` times over `original` positions keep their
    frequency, pairs that turn less than `slow` times are slowed by `factor`, a linear ramp in between."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class WindowLatentAttention:
    """weights: q [H (dn + dr), W], dkv [r + dr, W], dkv_norm [r], uk [H dn, r], uv [H dv, r], sink [H] (optional), o [W, H dv].
    Instead of q: dq [rq, W], dq_norm [rq], uq [H (dn + dr), rq] — queries from an RMS-normed latent of their own.
    g [H dv, W] (optional): the concatenated heads are multiplied by sigmoid(g h) ahead of the output projection.
    rot_freq: the frequency table (fp64, one per rotated pair), if not the YaRN table of rot_base / rot_scaling."""

    def __init__(self, weights: dict, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float, window,
                 rot_dims: int, rot_base: float, rot_scaling, eps: float, dtype, device, rot_freq=None):
        self.H, self.dn, self.dr, self.dv, self.r = heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.eps, self.dtype, self.device = float(scale), float(eps), dtype, device
        self.window = int(window) if window else 1 << 30
        self.rot_dims = int(rot_dims)
        if self.rot_dims > rot_dim or self.rot_dims % 2:
            raise ValueError("rotated dimensions must be even and at most rot_dim")
        freq, amp = yarn_table(self.rot_dims, rot_base, rot_scaling) if self.rot_dims else (torch.zeros(1, dtype=torch.float64), 1.0)
        if rot_freq is not None:
            freq, amp = rot_freq.to(torch.float64), 1.0
        self.freq, self.amp = freq.to(device), float(amp)
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        f = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.q_latent = "dq" in weights
        first = weights["dq"] if self.q_latent else weights["q"]
        self.q_cols = first.shape[0]                                               # q itself, or the query latent
        rows = [first, weights["dkv"]]
        self.gate_off = -1
        if "g" in weights:
            self.gate_off = self.q_cols + kv_rank + rot_dim
            rows.append(weights["g"])
        self.w_in = d(torch.cat(rows, 0))                                          # one projection: [q | latent | rotated key | gate]
        if self.q_latent:
            self.dq_norm, self.w_uq = f(weights["dq_norm"]), d(weights["uq"])
        self.dkv_norm = f(weights["dkv_norm"])
        self.sink = f(weights["sink"]) if "sink" in weights else None
        # absorbed key up-projection: q_abs[h] = q_nope[h] @ uk[h]  ->  stored [H, r, dn] for an A B^T product
        self.uk_t = d(weights["uk"].reshape(heads, dim, kv_rank).transpose(1, 2))
        self.uv = d(weights["uv"].reshape(heads, vdim, kv_rank))
        self.w_o = d(weights["o"])
        # long prompt portions in bfloat16 with 128 + 64 query / key dims and 128 value dims run the tcgen05 attention core of the MoE
        # prefill models (non-absorbed form: keys and values of the window are up-projected from the cached latents by one GEMM)
        self.tc_min_portion = 128
        self.tc_shape = dtype == torch.bfloat16 and dim == 128 and rot_dim == 64 and vdim == 128 and kv_rank % 64 == 0
        self.w_kv_up = d(torch.cat([weights["uk"], weights["uv"]], 0)) if self.tc_shape else None

    def cache_dims(self):
        return self.r, self.dr

    def forward(self, h: torch.Tensor, tb: ops.StepTables, ckv: torch.Tensor, kr: torch.Tensor, page_size: int) -> torch.Tensor:
        lib, T, H = ops.load(), h.shape[0], self.H
        proj_in = proj = lin(h, self.w_in, torch.float32)
        lat = None
        if self.q_latent:                         # q = uq rmsnorm(dq h); the latent and rotated key columns stay in proj_in
            proj = lin(ops.rms_rows(proj_in[:, :self.q_cols], self.dq_norm, self.eps, self.dtype), self.w_uq, torch.float32)
            lat = proj_in[:, self.q_cols:]
        ldp = proj.stride(0)
        s = torch.cuda.current_stream(h.device).cuda_stream
        dtc = ops.dt_code(ckv.dtype)
        ops.check(lib.kb2_seq_latent_prep(proj.data_ptr(), ldp, T, H, self.dn, self.dr, self.r, self.dkv_norm.data_ptr(), self.eps,
                                          self.freq.data_ptr(), self.rot_dims, self.amp, tb.positions.data_ptr(), tb.seq_of.data_ptr(),
                                          tb.pages.data_ptr(), tb.max_pages, page_size, ckv.data_ptr(), kr.data_ptr(), dtc, ops._ptr(lat),
                                          proj_in.stride(0), s))
        q = proj[:, :H * (self.dn + self.dr)].view(T, H, self.dn + self.dr)
        gated = self.gate_off >= 0
        o = torch.empty((T, H, self.dv), dtype=torch.float32 if gated else self.dtype, device=h.device)
        core = _core_lib() if self.tc_shape else False
        fast = [i for i, (_, n, _, _) in enumerate(tb.layout) if n >= self.tc_min_portion] if core else []
        if len(fast) < tb.S:
            q_abs = torch.empty((T, H, self.r), dtype=torch.float32, device=h.device)
            ops.gemm_heads(q[:, :, :self.dn], self.uk_t, q_abs)
            o_lat = torch.empty((T, H, self.r), dtype=torch.float32, device=h.device)
            # a step of few tokens (decoding) cuts each token's keys into pieces so that the whole GPU works on them
            blocks = T * ((H + 7) // 8)
            max_keys = max(min(self.window, start + n) for _, n, start, _ in tb.layout)
            nsplit = max(1, min(296 // max(blocks, 1), (max_keys + 31) // 32, 64))
            part_acc = torch.empty((T, nsplit, H, self.r), dtype=torch.float32, device=h.device) if nsplit > 1 else None
            part_ml = torch.empty((T, nsplit, H, 2), dtype=torch.float32, device=h.device) if nsplit > 1 else None
            ops.check(lib.kb2_seq_latent_window_attn(q_abs.data_ptr(), proj.data_ptr(), ldp, T, H, self.dn, self.dr, self.r, ckv.data_ptr(),
                                                     kr.data_ptr(), dtc, tb.positions.data_ptr(), tb.seq_of.data_ptr(), tb.pages.data_ptr(),
                                                     tb.max_pages, page_size, ops._ptr(self.sink), self.scale, self.window,
                                                     o_lat.data_ptr(), tb.cu.data_ptr() if fast else None, self.tc_min_portion, nsplit,
                                                     part_acc.data_ptr() if nsplit > 1 else None,
                                                     part_ml.data_ptr() if nsplit > 1 else None, s))
            ops.gemm_heads(o_lat, self.uv, o)
        for i in fast:
            from . import capi
            row0, n, start, _ = tb.layout[i]
            lo, rows = ops.key_rows(tb, i, self.window, page_size)
            kv_up = lin(ckv.view(-1, self.r).index_select(0, rows), self.w_kv_up, torch.bfloat16)     # [keys, H * (128 + 128)]
            kpe = kr.view(-1, self.dr).index_select(0, rows)
            q_bf = proj[row0:row0 + n, :H * (self.dn + self.dr)].to(torch.bfloat16).contiguous()
            o_rows = torch.empty((n, H, self.dv), dtype=torch.bfloat16, device=h.device) if gated else o[row0:row0 + n]
            capi.check(core.kb2_fmha_latent(q_bf.data_ptr(), kv_up.data_ptr(), kpe.data_ptr(), o_rows.data_ptr(), n, start - lo,
                                            start - lo + n, H, self.scale, min(self.window, 1 << 30), ops._ptr(self.sink),
                                            h.device.index or 0, s))
            if gated:
                o[row0:row0 + n].copy_(o_rows)
        if gated:
            o = ops.head_norm_gate(o.view(T, H * self.dv), H, self.dv, self.dtype, gate=proj_in[:, self.gate_off:], gate_act="sigmoid")
        return lin(o.view(T, H * self.dv), self.w_o, torch.float32)


class GatedDeltaMixer:
    """weights: q, k [Hk dk, W], v, g [H dv, W], a, b [H, W], q_conv, k_conv, v_conv [channels, taps], A_log, dt_bias [H],
    norm [dv], o [W, H dv]."""

    def __init__(self, weights: dict, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float, dtype, device):
        self.H, self.Hk, self.dk, self.dv, self.K = heads, kv_heads, dim, vdim, int(taps)
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.eps, self.dtype, self.device = float(eps), dtype, device
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        f = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.C = 2 * kv_heads * dim + heads * vdim                                  # convolved channels: q | k | v
        self.g_off, self.a_off, self.b_off = self.C, self.C + heads * vdim, self.C + heads * vdim + heads
        self.w_in = d(torch.cat([weights[k] for k in ("q", "k", "v", "g", "a", "b")], 0))
        self.taps = f(torch.cat([weights["q_conv"], weights["k_conv"], weights["v_conv"]], 0))
        self.A_log, self.dt_bias, self.norm = f(weights["A_log"]), f(weights["dt_bias"]), f(weights["norm"])
        self.w_o = d(weights["o"])
        # key sizes 32 / 64 / 128 with value sizes that are multiples of 32 keep the state in registers; others in shared memory
        self.register_state_kernel = dim in (32, 64, 128) and vdim % 32 == 0

    def register_state(self, pool):
        """(conv tail [slots, C, taps - 1], recurrent state [slots, H, dk, dv]) in a RecurrentStatePool."""
        return pool.register(self.C, max(self.K - 1, 1)), pool.register(self.H, self.dk, self.dv)

    def forward(self, h: torch.Tensor, tb: ops.StepTables, tail: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        lib, T = ops.load(), h.shape[0]
        proj = lin(h, self.w_in, torch.float32)
        s = torch.cuda.current_stream(h.device).cuda_stream
        conv = torch.empty((T, self.C), dtype=torch.float32, device=h.device)
        ops.check(lib.kb2_seq_conv_silu(proj.data_ptr(), proj.stride(0), T, tb.S, self.C, self.K, self.taps.data_ptr(), tail.data_ptr(),
                                        tb.seq_of.data_ptr(), tb.cu.data_ptr(), tb.slots.data_ptr(), conv.data_ptr(), s))
        o = torch.empty((T, self.H * self.dv), dtype=self.dtype, device=h.device)
        scratch = None
        if self.register_state_kernel or self.dk * self.dv > 32768:      # a large state is cut into column slices that meet in scratch
            scratch = torch.empty(2 * T * self.Hk * self.dk + 2 * T * self.H + T * self.H * self.dv + 4, dtype=torch.float32, device=h.device)
        ops.check(lib.kb2_seq_delta_rule(conv.data_ptr(), self.C, proj.data_ptr(), proj.stride(0), self.g_off, self.a_off, self.b_off, T,
                                         tb.S, self.H, self.Hk, self.dk, self.dv, self.A_log.data_ptr(), self.dt_bias.data_ptr(),
                                         self.norm.data_ptr(), self.eps, state.data_ptr(), tb.cu.data_ptr(), tb.slots.data_ptr(),
                                         scratch.data_ptr() if scratch is not None else None, o.data_ptr(), ops.dt_code(self.dtype), s))
        return lin(o, self.w_o, torch.float32)


def lin_cols(proj: torch.Tensor, off: int, r: int, w: torch.Tensor, dtype) -> torch.Tensor:
    """Second factor of a low-rank projection on columns [off, off + r) of an fp32 product: fp32 out.  The generic kernel reads the
    strided fp32 columns as they are; only a long bfloat16 step with a rank the tensor-core kernel takes is rounded and packed."""
    a = proj[:, off:off + r]
    if dtype == torch.bfloat16 and proj.shape[0] >= 256 and r % 64 == 0 and _core_lib():
        return lin(a.to(torch.bfloat16).contiguous(), w, torch.float32)
    return ops.gemm(a, w, torch.float32)


class GatedLinearAttention:
    """weights: q, k [H dk, W], v, g [H dv, W], a1 [r, W], a2 [H dk, r], a2_b [H dk], norm [dv], o [W, H dv].

    Per token and head: alpha = sigmoid(a2 (a1 h) + a2_b)^(1 / tau), one decay per key channel; S <- diag(alpha) S + k v^T;
    o = S^T (q dk^-1/2); out = o / rms(o) * norm * silu(g h), heads side by side, then the output projection.  The state
    [slots, H, dk, dv], the decays and their logarithms are fp32."""

    def __init__(self, weights: dict, heads: int, dim: int, vdim: int, tau: float, eps: float, dtype, device, q_scale=None):
        self.H, self.dk, self.dv, self.tau = heads, dim, vdim, float(tau)
        self.q_scale = float(dim) ** -0.5 if q_scale is None else float(q_scale)
        self.eps, self.dtype, self.device = float(eps), dtype, device
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        f = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.ra = weights["a1"].shape[0]
        self.q_off, self.k_off, self.v_off = 0, heads * dim, 2 * heads * dim
        self.g_off = self.v_off + heads * vdim
        self.a_off = self.g_off + heads * vdim
        rows = [weights[k] for k in ("q", "k", "v", "g", "a1")]
        pad = -sum(r.shape[0] for r in rows) % 4                                              # rows of the product start on 16 bytes
        if pad:
            rows.append(torch.zeros(pad, rows[0].shape[1], dtype=rows[0].dtype))
        self.w_in = d(torch.cat(rows, 0))                                                     # one projection of the layer input
        self.w_a2, self.a2_b, self.norm = d(weights["a2"]), f(weights["a2_b"]), f(weights["norm"])
        if self.w_a2.shape[0] != heads * dim or self.a2_b.numel() != heads * dim or self.norm.numel() != vdim:
            raise ValueError("decay projection / norm do not match heads x dim / vdim")
        self.w_o = d(weights["o"])
        self.register_state_kernel = dim in (32, 64, 128, 256) and vdim % 32 == 0

    def register_state(self, pool):
        """Recurrent state [slots, H, dk, dv] in a RecurrentStatePool."""
        return pool.register(self.H, self.dk, self.dv)

    def forward(self, h: torch.Tensor, tb: ops.StepTables, state: torch.Tensor) -> torch.Tensor:
        lib, T, H = ops.load(), h.shape[0], self.H
        proj = lin(h, self.w_in, torch.float32)
        dec_in = lin_cols(proj, self.a_off, self.ra, self.w_a2, self.dtype)                   # [T, H dk]
        o = torch.empty((T, H * self.dv), dtype=torch.float32, device=h.device)
        # key sizes 32 / 64 / 128 / 256 with value sizes that are multiples of 32 keep the state in registers (the decays meet in scratch)
        scratch = torch.empty((T, H * self.dk), dtype=torch.float32, device=h.device) if self.register_state_kernel else None
        ops.check(lib.kb2_seq_gla(proj.data_ptr(), proj.stride(0), self.q_off, self.k_off, self.v_off, dec_in.data_ptr(), dec_in.stride(0),
                                  self.a2_b.data_ptr(), self.tau, self.q_scale, T, tb.S, H, self.dk, self.dv, state.data_ptr(),
                                  tb.cu.data_ptr(), tb.slots.data_ptr(), ops._ptr(scratch), o.data_ptr(),
                                  torch.cuda.current_stream(h.device).cuda_stream))
        o = ops.head_norm_gate(o, H, self.dv, self.dtype, norm=self.norm, eps=self.eps, gate=proj[:, self.g_off:], gate_act="silu")
        return lin(o, self.w_o, torch.float32)


class SelectiveScan:
    """weights: in [2 C, W] (x | z), conv [C, taps], conv_b [C], x [R + 2 N, C] (dt | B | C), dt [C, R], dt_b [C], A_log [C, N], D [C],
    o [W, C].

    x = silu(causal conv(in h)[:C] + conv_b); dt = softplus(dt (x x)[:R] + dt_b) per channel; per channel c and state n:
    S <- exp(dt_c A[c, n]) S + dt_c x_c B_n with A = -exp(A_log); y_c = sum_n S[c, n] C_n + D_c x_c; out = o (y silu(z)).
    The state [slots, C, N], the convolution's last taps - 1 inputs, step sizes and exponentials are fp32."""

    def __init__(self, weights: dict, inner: int, state: int, dt_rank: int, taps: int, dtype, device):
        self.C, self.N, self.R, self.K = int(inner), int(state), int(dt_rank), int(taps)
        self.dtype, self.device = dtype, device
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        f = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.w_in, self.w_x, self.w_dt, self.w_o = d(weights["in"]), d(weights["x"]), d(weights["dt"]), d(weights["o"])
        self.taps, self.conv_b = f(weights["conv"]), f(weights["conv_b"])
        self.dt_b, self.A_log, self.D = f(weights["dt_b"]), f(weights["A_log"]), f(weights["D"])
        if (self.w_in.shape[0] != 2 * self.C or self.w_x.shape != (self.R + 2 * self.N, self.C) or self.taps.shape != (self.C, self.K)
                or self.A_log.shape != (self.C, self.N)):
            raise ValueError("selective scan: tensor shapes do not match inner / state / dt_rank / taps")

    def register_state(self, pool):
        """(conv tail [slots, C, taps - 1], state [slots, C, N]) in a RecurrentStatePool."""
        return pool.register(self.C, max(self.K - 1, 1)), pool.register(self.C, self.N)

    def forward(self, h: torch.Tensor, tb: ops.StepTables, tail: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        lib, T = ops.load(), h.shape[0]
        proj = lin(h, self.w_in, torch.float32)                                               # [T, x: C | z: C]
        xc = ops.conv(proj, self.C, self.taps, self.conv_b, True, tail, tb, bias_after=True)  # [T, C] fp32
        big = self.dtype == torch.bfloat16 and T >= 256 and bool(_core_lib())
        xp = lin(xc.to(torch.bfloat16) if big else xc, self.w_x, torch.float32, min_n=16)     # [T, dt: R | B: N | C: N]
        dt_in = lin_cols(xp, 0, self.R, self.w_dt, self.dtype)                                # [T, C]
        y = torch.empty((T, self.C), dtype=self.dtype, device=h.device)
        ops.check(lib.kb2_seq_selective_scan(xc.data_ptr(), xc.stride(0), dt_in.data_ptr(), dt_in.stride(0), self.dt_b.data_ptr(),
                                             xp.data_ptr(), xp.stride(0), self.R, proj.data_ptr(), proj.stride(0), self.C,
                                             self.A_log.data_ptr(), self.D.data_ptr(), T, tb.S, self.C, self.N, state.data_ptr(),
                                             tb.cu.data_ptr(), tb.slots.data_ptr(), y.data_ptr(), ops.dt_code(self.dtype),
                                             torch.cuda.current_stream(h.device).cuda_stream))
        return lin(y, self.w_o, torch.float32)


class SideBySide:
    """Two mixers read the same input; the result is coef (left / rms(left) * w_left + right / rms(right) * w_right) over the width."""

    def __init__(self, left, right, w_left: torch.Tensor, w_right: torch.Tensor, eps: float, device, coef: float = 0.5):
        self.left, self.right, self.eps, self.coef = left, right, float(eps), float(coef)
        self.w_left = w_left.to(device=device, dtype=torch.float32).contiguous()
        self.w_right = w_right.to(device=device, dtype=torch.float32).contiguous()

    def merge(self, y_left: torch.Tensor, y_right: torch.Tensor) -> torch.Tensor:
        return ops.branch_merge(y_left, y_right, self.w_left, self.w_right, self.eps, self.coef)


class ChannelDeltaMixer:
    """Gated delta rule whose decay is one number per head and key channel.
    weights: q, k [Hk dk, W], v [H dv, W], b [H, W], a1 [r, W], a2 [H dk, r], g1 [r', W], g2 [H dv, r'], q_conv, k_conv, v_conv
    [channels, taps], A_log [H], dt_bias [H dk], norm [dv], o [W, H dv].

    Per token: q, k, v = silu(conv(projection)); q and k unit vectors per head (q also times dk^-1/2); beta = sigmoid(b h);
    g = exp(-exp(A_log[h]) softplus(a2 (a1 h) + dt_bias)) per (head, key channel); S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q; out = o / rms(o) * norm * sigmoid(g2 (g1 h)), then the output projection.  State and everything that feeds the recurrence
    are fp32."""

    def __init__(self, weights: dict, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float, dtype, device):
        self.H, self.Hk, self.dk, self.dv, self.K = heads, kv_heads, dim, vdim, int(taps)
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.eps, self.dtype, self.device = float(eps), dtype, device
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        f = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.C = 2 * kv_heads * dim + heads * vdim                                  # convolved channels: q | k | v
        self.ra, self.rg = weights["a1"].shape[0], weights["g1"].shape[0]
        self.b_off, self.a_off, self.g_off = self.C, self.C + heads, self.C + heads + self.ra
        self.w_in = d(torch.cat([weights[k] for k in ("q", "k", "v", "b", "a1", "g1")], 0))     # one projection of the layer input
        self.w_a2, self.w_g2 = d(weights["a2"]), d(weights["g2"])
        self.taps = f(torch.cat([weights["q_conv"], weights["k_conv"], weights["v_conv"]], 0))
        self.A_log, self.dt_bias, self.norm = f(weights["A_log"]), f(weights["dt_bias"]), f(weights["norm"])
        if self.dt_bias.numel() != heads * dim or self.w_a2.shape[0] != heads * dim or self.w_g2.shape[0] != heads * vdim:
            raise ValueError("decay / gate projections do not match heads x dim / heads x vdim")
        self.w_o = d(weights["o"])
        self.register_state_kernel = dim in (32, 64, 128) and vdim % 32 == 0

    def register_state(self, pool):
        """(conv tail [slots, C, taps - 1], recurrent state [slots, H, dk, dv]) in a RecurrentStatePool."""
        return pool.register(self.C, max(self.K - 1, 1)), pool.register(self.H, self.dk, self.dv)

    def _second(self, proj, off, r, w):
        """Second factor of a low-rank projection on columns [off, off + r) of the fp32 first product.  The generic kernel reads the
        strided fp32 columns as they are; only a long bfloat16 step with a rank the tensor-core kernel takes is rounded and packed."""
        a = proj[:, off:off + r]
        if self.dtype == torch.bfloat16 and proj.shape[0] >= 256 and r % 64 == 0 and _core_lib():
            return lin(a.to(torch.bfloat16).contiguous(), w, torch.float32)
        return ops.gemm(a, w, torch.float32)

    def forward(self, h: torch.Tensor, tb: ops.StepTables, tail: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        lib, T, H = ops.load(), h.shape[0], self.H
        proj = lin(h, self.w_in, torch.float32)
        s = torch.cuda.current_stream(h.device).cuda_stream
        conv = ops.conv(proj, self.C, self.taps, None, True, tail, tb)
        dec_in = self._second(proj, self.a_off, self.ra, self.w_a2)                 # [T, H dk]
        gate_in = self._second(proj, self.g_off, self.rg, self.w_g2)                # [T, H dv]
        o = torch.empty((T, H * self.dv), dtype=self.dtype, device=h.device)
        scratch = None
        if self.register_state_kernel or self.dk * self.dv > 32768:      # a large state is cut into column slices that meet in scratch
            n = 2 * T * self.Hk * self.dk + T * H + T * H * self.dk + T * H * self.dv + 16
            scratch = torch.empty(n, dtype=torch.float32, device=h.device)
        beta_in = proj[:, self.b_off:]
        ops.check(lib.kb2_seq_delta_rule_ch(conv.data_ptr(), self.C, beta_in.data_ptr(), proj.stride(0), dec_in.data_ptr(), dec_in.stride(0),
                                            gate_in.data_ptr(), gate_in.stride(0), 1, T, tb.S, H, self.Hk, self.dk, self.dv,
                                            self.A_log.data_ptr(), self.dt_bias.data_ptr(), self.norm.data_ptr(), self.eps,
                                            state.data_ptr(), tb.cu.data_ptr(), tb.slots.data_ptr(), ops._ptr(scratch), o.data_ptr(),
                                            ops.dt_code(self.dtype), s))
        return lin(o, self.w_o, torch.float32)


class GatedMLP:
    """weights: gate, up [F, W], down [W, F].  act: "gelu_tanh" (gelu(g) u), "silu" (silu(g) u) or "clamped_swish"
    (g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit)).  gated False: weights up, down only and
    down(act(up h)) with act "relu2" (the square of relu)."""

    KINDS = {"gelu_tanh": ops.GLU_GELU_TANH, "silu": ops.GLU_SILU, "clamped_swish": ops.GLU_CLAMPED_SWISH, "relu2": ops.ACT_RELU2}

    def __init__(self, weights: dict, dtype, device, act: str = "gelu_tanh", limit: float = 0.0, alpha: float = 1.0, gated: bool = True):
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        if gated == (act == "relu2"):
            raise ValueError("relu2 is the activation of the ungated form, and its only one")
        self.w_gu = d(torch.cat([weights["gate"], weights["up"]], 0)) if gated else d(weights["up"])
        self.w_down, self.dtype = d(weights["down"]), dtype
        self.kind, self.limit, self.alpha = self.KINDS[act], float(limit), float(alpha)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        gu = lin(h, self.w_gu, self.dtype)
        a = ops.act_mul(gu, self.dtype) if self.kind == ops.GLU_GELU_TANH else ops.glu(gu, self.dtype, self.kind, self.limit, self.alpha)
        return lin(a, self.w_down, torch.float32)


def rotary_table(dims: int, base: float, factor: float = 1.0) -> torch.Tensor:
    """Angular frequency of each rotated pair (fp64): base^(-2i / dims) / factor (linear position scaling)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims) / float(factor)


def llama3_table(dims: int, base: float, scaling=None) -> torch.Tensor:
    """Angular frequency of each rotated pair (fp64), base^(-2i / dims), rescaled by wavelength l = 2 pi / f against a training length
    `original`: kept where l < original / high, divided by `factor` where l > original / low, and in between blended as
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low).  scaling = {factor, low, high, original} or None."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if not scaling:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    wave = 2.0 * math.pi / f
    if high == low:
        return torch.where(wave > orig / low, f / factor, f)
    sm = (orig / wave - low) / (high - low)
    mid = (1.0 - sm) * f / factor + sm * f
    return torch.where(wave < orig / high, f, torch.where(wave > orig / low, f / factor, mid))


class MultiMapAttention:
    """weights: q [H M d, W], k [G M d, W], v [G dv, W] (each with an optional bias `<name>_b`), q_norm / k_norm [d] (optional RMS norm
    weights, shared by heads and maps), g [H, W] (optional output gate), o [W, H dv].  Rows of q and k are laid out head by head as
    [map 0, map 1, ...].  own_kv False: no k / v tensors, the layer reads the cache pools it is given.

    A head's output is sum_m map_coef[m] * softmax(q_m k_m^T scale) v over the visible keys (same chunk of `chunk` positions counted
    from position 0, at most `window` back, causal); with unit_norm it is divided by its root mean square and multiplied by
    post_scale; with a gate it is multiplied by sigmoid(g h).

    conv_taps > 0: q_conv / k_conv / v_conv [channels, taps] — a short causal convolution over time on every channel of the biased
    projections, ahead of norm and rotation; its last taps - 1 inputs per sequence live in a state slot (`register_state`).
    norm_whole: q_norm / k_norm have the size of the whole projection and one root mean square is taken over all of q (of k).
    rot_half: dimension i turns with i + rot_dims / 2 (default: 2i with 2i + 1).  rot_freq: the frequency table, if not
    base^(-2i / dims) / rot_factor.  softcap > 0: a scaled score s becomes softcap tanh(s / softcap).

    sink [H] (optional weight): exp(sink_h) joins the softmax denominator of head h (no key, no value, not scaled).
    pool > 0 (with a window): beside the window's keys a position sees one key and value per block of `pool` positions that lies wholly
    before its window — the means of the block's cached keys and values, kept in pooled pools (`forward(..., pooled=(kp, vp))`).
    rot_values: values are cached rotated by their positions over all of vdim (pair m by position * rot_base^(-2m / vdim), no factor,
    the pair layout of the keys) and each head's output is turned back by the query's position, ahead of the gate.
    gate_per_element: g is [H dv, W], one sigmoid gate per output element (default [H, W]: one per head)."""

    def __init__(self, weights: dict, heads: int, kv_heads: int, maps: int, dim: int, vdim: int, scale: float, eps: float, dtype, device,
                 chunk=None, window=None, rot_dims: int = 0, rot_base: float = 10000.0, rot_factor: float = 1.0, map_coef=None,
                 unit_norm: bool = False, post_scale: float = 1.0, own_kv: bool = True, conv_taps: int = 0, norm_whole: bool = False,
                 rot_half: bool = False, rot_freq=None, softcap: float = 0.0, pool: int = 0, rot_values: bool = False,
                 gate_per_element: bool = False):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if rot_dims > dim or rot_dims % 2:
            raise ValueError("rotated dimensions must be even and at most dim")
        self.H, self.G, self.M, self.d, self.dv = heads, kv_heads, int(maps), dim, vdim
        self.scale, self.eps, self.dtype, self.device, self.own_kv = float(scale), float(eps), dtype, device, bool(own_kv)
        self.chunk = int(chunk) if chunk else 0
        self.window = int(window) if window else 1 << 30
        self.rot_dims = int(rot_dims)
        self.freq = rotary_table(self.rot_dims, rot_base, rot_factor).to(device) if self.rot_dims else None
        if self.rot_dims and rot_freq is not None:
            if rot_freq.numel() != self.rot_dims // 2:
                raise ValueError("one frequency per rotated pair")
            self.freq = rot_freq.to(device=device, dtype=torch.float64).contiguous()
        self.norm_whole, self.rot_half, self.softcap, self.K = bool(norm_whole), bool(rot_half), float(softcap or 0.0), int(conv_taps or 0)
        if self.K and not own_kv:
            raise ValueError("the convolution needs projections of the layer's own")
        self.unit_norm, self.post_scale = bool(unit_norm), float(post_scale)
        self.pool, self.gate_wide = int(pool or 0), bool(gate_per_element)
        if self.pool and (self.chunk or not window or not own_kv):
            raise ValueError("pooled blocks need a sliding window, no chunks and a cache of the layer's own")
        if rot_values and vdim % 2:
            raise ValueError("rotated values need an even value size")
        self.vfreq = rotary_table(vdim, rot_base, 1.0).to(device) if rot_values else None
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        f = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.sink = f(weights["sink"]) if "sink" in weights else None
        if self.sink is not None and self.sink.numel() != heads:
            raise ValueError("one sink per head")
        self.map_coef = f(torch.as_tensor(map_coef, dtype=torch.float64)) if map_coef is not None else None
        if self.map_coef is not None and self.map_coef.numel() != self.M:
            raise ValueError("one coefficient per map")
        names = ["q"] + (["k", "v"] if own_kv else [])
        rows = [weights[n] for n in names]
        self.gate_off = sum(r.shape[0] for r in rows) if "g" in weights else -1
        if "g" in weights:
            rows.append(weights["g"])
        self.w_in = d(torch.cat(rows, 0))                                   # one projection: [q | k | v | gate]
        if any(n + "_b" in weights for n in names):
            self.bias = f(torch.cat([weights.get(n + "_b", torch.zeros(weights[n].shape[0])).float() for n in names], 0))
        else:
            self.bias = None
        self.q_norm = f(weights["q_norm"]) if "q_norm" in weights else None
        self.k_norm = f(weights["k_norm"]) if (own_kv and "k_norm" in weights) else None
        self.w_o = d(weights["o"])
        self.C = sum(weights[n].shape[0] for n in names)                    # q | k | v columns of the projection
        self.taps = f(torch.cat([weights[n + "_conv"] for n in names], 0)) if self.K else None
        for nm, w, n in (("q", self.q_norm, heads * maps * dim), ("k", self.k_norm, kv_heads * maps * dim)):
            if w is not None and w.numel() != (n if norm_whole else dim):
                raise ValueError(f"{nm}_norm has {w.numel()} weights")
        # long prompt portions in bfloat16 with 128 query / key dims per map and 128 or 256 value dims run the tcgen05 attention core of
        # the MoE prefill models, one call per chunk the portion touches, on keys and values gathered from the pages
        self.tc_min_portion = 128
        # (a sink goes into the core's softmax; pooled blocks are a second pass on the plain kernel, merged by the two log-sum-exps)
        self.tc_shape = dtype == torch.bfloat16 and dim == 128 and vdim in (128, 256) and (self.M == 1 or (self.sink is None and not self.pool))

    def cache_dims(self):
        """(key width, value width) of a cache row; with pooled blocks a third entry, the block length."""
        return (self.G * self.M * self.d, self.G * self.dv) + ((self.pool,) if self.pool else ())

    def register_state(self, pool):
        """Convolution tail [slots, C, taps - 1] in a RecurrentStatePool (None without a convolution)."""
        return pool.register(self.C, max(self.K - 1, 1)) if self.K else None

    def _tensor_core_portion(self, core, proj, a, tb, i, kc, vc, page_size, stream, lse=None):
        """Sequence i of the step on the tcgen05 kernel: a[rows of the portion] = per-map attention outputs (fp32)."""
        import numpy as np
        from . import capi
        row0, n, start, pages = tb.layout[i]
        H, G, M, d, dv, chunk = self.H, self.G, self.M, self.d, self.dv, self.chunk
        first = start // chunk * chunk if chunk else 0
        first = max(first, start - self.window + 1)
        key = ("rows_from", i, first, page_size)                  # the layers of a step share the row list of a sequence
        if key not in tb._key_rows:
            j = np.arange(first, start + n, dtype=np.int64)
            host = torch.from_numpy(np.asarray(pages, dtype=np.int64)[j // page_size] * page_size + j % page_size)
            tb._key_rows[key] = host.to(proj.device, non_blocking=True)
        rows = tb._key_rows[key]
        k_rows = kc.view(-1, G * M * d).index_select(0, rows)
        v_rows = vc.view(-1, G * dv).index_select(0, rows)
        q = proj[row0:row0 + n, :H * M * d].to(torch.bfloat16).contiguous()
        pos = start
        while pos < start + n:
            cstart = pos // chunk * chunk if chunk else 0
            end = min(start + n, cstart + chunk) if chunk else start + n
            lo = max(cstart, first)
            m = end - pos
            if self.sink is not None or lse is not None:
                capi.check(core.kb2_fmha_maps_sink(q[pos - start:].data_ptr(), k_rows[lo - first:].data_ptr(), v_rows[lo - first:].data_ptr(),
                                                   a[row0 + pos - start:].data_ptr(), m, pos - lo, end - lo, H * M, G, M, dv, self.scale,
                                                   self.softcap, min(self.window, 1 << 30), ops._ptr(self.sink),
                                                   lse[row0 + pos - start:].data_ptr() if lse is not None else None,
                                                   proj.device.index or 0, stream))
            else:
                capi.check(core.kb2_fmha_maps_softcap(q[pos - start:].data_ptr(), k_rows[lo - first:].data_ptr(), v_rows[lo - first:].data_ptr(),
                                                      a[row0 + pos - start:].data_ptr(), m, pos - lo, end - lo, H * M, G, M, dv, self.scale,
                                                      self.softcap, min(self.window, 1 << 30), proj.device.index or 0, stream))
            pos = end

    def forward(self, h: torch.Tensor, tb: ops.StepTables, kc: torch.Tensor, vc: torch.Tensor, page_size: int, tail=None, pooled=None) -> torch.Tensor:
        lib, T, H, G, M = ops.load(), h.shape[0], self.H, self.G, self.M
        if self.pool and pooled is None:
            raise ValueError("this layer needs its pooled pools")
        kp, vp = pooled if self.pool else (None, None)
        proj_in = proj = lin(h, self.w_in, torch.float32)
        bias = self.bias
        if self.K:                                   # q | k | v through the convolution (bias first); the gate columns stay in proj_in
            proj, bias = ops.conv(proj_in, self.C, self.taps, self.bias, False, tail, tb), None
        ldp = proj.stride(0)
        s = torch.cuda.current_stream(h.device).cuda_stream
        dtc = ops.dt_code(kc.dtype)
        ops.check(lib.kb2_seq_head_kv_prep(proj.data_ptr(), ldp, T, H, G if self.own_kv else 0, M, self.d, self.dv, ops._ptr(bias),
                                           ops._ptr(self.q_norm), ops._ptr(self.k_norm), self.eps, ops._ptr(self.freq), self.rot_dims,
                                           tb.positions.data_ptr(), tb.seq_of.data_ptr(), tb.pages.data_ptr(), tb.max_pages, page_size,
                                           kc.data_ptr(), vc.data_ptr(), dtc, int(self.norm_whole), int(self.rot_half), ops._ptr(self.vfreq), s))
        if self.pool:                                # the tokens that complete a block write its mean key and value
            ops.check(lib.kb2_seq_kv_pool(kc.data_ptr(), vc.data_ptr(), kp.data_ptr(), vp.data_ptr(), dtc, G * M * self.d, G * self.dv, self.pool,
                                          T, tb.positions.data_ptr(), tb.seq_of.data_ptr(), tb.pages.data_ptr(), tb.max_pages, page_size, s))
        # a step of few tokens (decoding) cuts each token's keys into pieces so that the whole GPU works on them
        reach = min(self.window, self.chunk) if self.chunk else self.window
        max_keys = max(min(reach, start + n) + ((start + n) // self.pool if self.pool else 0) for _, n, start, _ in tb.layout)
        nsplit = max(1, min(296 // max(T * G, 1), (max_keys + 31) // 32, 64))
        core = _core_lib() if self.tc_shape else False
        fast = [i for i, (_, n, _, _) in enumerate(tb.layout) if n >= self.tc_min_portion] if core else []
        if fast:
            nsplit = 1
        a = part_acc = part_ml = None
        if nsplit > 1:
            part_acc = torch.empty((T * H * M, nsplit, self.dv), dtype=torch.float32, device=h.device)
            part_ml = torch.empty((T * H * M, nsplit, 2), dtype=torch.float32, device=h.device)
            a = part_acc                                                     # unused by the kernels when the range is cut
        else:
            a = torch.empty((T, H, M, self.dv), dtype=torch.float32, device=h.device)
        if len(fast) < tb.S:
            ops.check(lib.kb2_seq_paged_attn(proj.data_ptr(), ldp, T, H, G, M, self.d, self.dv, kc.data_ptr(), vc.data_ptr(), dtc,
                                             tb.positions.data_ptr(), tb.seq_of.data_ptr(), tb.pages.data_ptr(), tb.max_pages, page_size,
                                             self.scale, self.chunk, min(self.window, 1 << 30), a.data_ptr(), nsplit, ops._ptr(part_acc),
                                             ops._ptr(part_ml), tb.cu.data_ptr() if fast else None, self.tc_min_portion, self.softcap,
                                             ops._ptr(self.sink), self.pool, ops._ptr(kp), ops._ptr(vp), 0, s))
        lse = torch.empty((T, H), dtype=torch.float32, device=h.device) if (fast and self.pool) else None
        for i in fast:
            self._tensor_core_portion(core, proj, a, tb, i, kc, vc, page_size, s, lse=lse)
        if fast and self.pool:                       # the pooled blocks of the long portions: a second pass, joined by the log-sum-exps
            p_acc = torch.empty((T * H, self.dv), dtype=torch.float32, device=h.device)
            p_ml = torch.empty((T * H, 2), dtype=torch.float32, device=h.device)
            ops.check(lib.kb2_seq_paged_attn(proj.data_ptr(), ldp, T, H, G, M, self.d, self.dv, kc.data_ptr(), vc.data_ptr(), dtc,
                                             tb.positions.data_ptr(), tb.seq_of.data_ptr(), tb.pages.data_ptr(), tb.max_pages, page_size,
                                             self.scale, 0, min(self.window, 1 << 30), a.data_ptr(), 1, p_acc.data_ptr(), p_ml.data_ptr(),
                                             tb.cu.data_ptr(), self.tc_min_portion, self.softcap, None, self.pool, kp.data_ptr(),
                                             vp.data_ptr(), 1, s))
            ops.check(lib.kb2_seq_pool_merge(a.data_ptr(), lse.data_ptr(), p_acc.data_ptr(), p_ml.data_ptr(), T, H, self.dv,
                                             tb.seq_of.data_ptr(), tb.cu.data_ptr(), self.tc_min_portion, s))
        o = torch.empty((T, H * self.dv), dtype=self.dtype, device=h.device)
        gate = proj_in[:, self.gate_off:] if self.gate_off >= 0 else None
        ops.check(lib.kb2_seq_attn_finish(a.data_ptr(), ops._ptr(part_acc), ops._ptr(part_ml), nsplit, T, H, M, self.dv, ops._ptr(self.map_coef),
                                          int(self.unit_norm), self.eps, self.post_scale, ops._ptr(gate), proj_in.stride(0), o.data_ptr(),
                                          ops.dt_code(self.dtype), None, None, 0, int(self.gate_wide), tb.positions.data_ptr(),
                                          ops._ptr(self.vfreq), int(self.rot_half), s))
        return lin(o, self.w_o, torch.float32)


class RoutedExperts:
    """weights: router [E + identity, W], correction [E + identity] (optional), e<i>_gate / e<i>_up [F, W], e<i>_down [W, F] for i < E,
    shared_gate / shared_up / shared_down (optional shared expert of the same form, run for every token and added), shared_sg [1, W]
    (optional: the shared expert's output is multiplied by sigmoid(shared_sg h), one number per token).
    gated False: the experts (and the shared one) have no gate tensor and compute down(act(up h)); act: "silu" (gated) or "relu2".

    Scores are softmax (or sigmoid) of the fp32 router logits over all E + identity outputs; the choice adds `correction`; the outputs
    form `groups` equal groups of neighbours of which the `keep` with the largest group score stay eligible (group_score "max": the
    group's largest choice, "top2": the sum of its two largest); the `top` largest choices are taken and weighted by their scores
    (divided by their sum if `renorm`, times out_scale).  The last `identity` outputs are identity experts: they return their input."""

    def __init__(self, weights: dict, experts: int, identity: int, top: int, dtype, device, groups: int = 1, keep: int = 1,
                 score: str = "softmax", renorm: bool = False, out_scale: float = 1.0, gated: bool = True, act: str = "silu",
                 group_score: str = "max"):
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        self.E, self.ident, self.top, self.groups, self.keep = int(experts), int(identity), int(top), int(groups), int(keep)
        self.score, self.renorm, self.out_scale, self.dtype, self.device = score, bool(renorm), float(out_scale), dtype, device
        self.gated, self.group_score = bool(gated), group_score
        if gated == (act == "relu2") or act not in ("silu", "relu2") or group_score not in ("max", "top2"):
            raise ValueError("experts: silu with a gate or relu2 without; group_score max or top2")
        self.act_kind = ops.GLU_SILU if gated else ops.ACT_RELU2
        if weights["router"].shape[0] != self.E + self.ident:
            raise ValueError("router rows must equal experts + identity experts")
        if (self.E + self.ident) % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError("expert groups must divide experts + identity experts, 1 <= keep <= groups")
        rows = [weights["router"]]
        self.sg_col = -1
        if "shared_sg" in weights:                  # the shared expert's gate rides on the router product as one more column
            self.sg_col = self.E + self.ident
            rows.append(weights["shared_sg"].reshape(1, -1))
            pad = -(self.sg_col + 1) % 16           # a width the tensor-core product takes
            if pad:
                rows.append(torch.zeros(pad, weights["router"].shape[1], dtype=weights["router"].dtype))
        self.w_router = d(torch.cat(rows, 0))
        self.correction = weights["correction"].to(device=device, dtype=torch.float32).contiguous() if "correction" in weights else None
        if self.E:
            first = (lambda i: torch.cat([weights[f"e{i}_gate"], weights[f"e{i}_up"]], 0)) if gated else (lambda i: weights[f"e{i}_up"])
            self.w_gu = d(torch.stack([first(i) for i in range(self.E)], 0))                         # [E, 2F | F, W]
            self.w_down = d(torch.stack([weights[f"e{i}_down"] for i in range(self.E)], 0))          # [E, W, F]
            self.F = self.w_down.shape[2]
        self.shared = GatedMLP({k[len("shared_"):]: v for k, v in weights.items() if k.startswith("shared_") and k != "shared_sg"}, dtype,
                               device, act=act, gated=gated) if "shared_up" in weights else None
        self.tile = ops.load().kb2_seq_moe_tile_rows()
        self.gemv_max_tokens = 8
        # bfloat16 steps that bring at least this many rows per expert on average run on the grouped tcgen05 GEMM (128-row tiles)
        self.tc_min_rows_per_expert = 16

    def _bin(self, ids, slots, tile):
        """Device tables of the binned order with runs padded to `tile` rows (see kb2_seq_moe_bin)."""
        E, dev = self.E, ids.device
        max_rows = (slots + E * (tile - 1) + tile - 1) // tile * tile
        max_tiles = max_rows // tile
        ints = torch.empty(3 * E + 2 + max_tiles + max_rows + slots, dtype=torch.int32, device=dev)
        t = {"counts": ints[:E], "offs": ints[E:2 * E + 1], "cursor": ints[2 * E + 1:3 * E + 1], "n_tiles": ints[3 * E + 1:3 * E + 2],
             "tile_expert": ints[3 * E + 2:3 * E + 2 + max_tiles], "slot_row": ints[3 * E + 2 + max_tiles:3 * E + 2 + max_tiles + max_rows],
             "pos": ints[3 * E + 2 + max_tiles + max_rows:], "max_rows": max_rows, "max_tiles": max_tiles}
        ops.check(ops.load().kb2_seq_moe_bin(ids.data_ptr(), slots, E, tile, t["counts"].data_ptr(), t["offs"].data_ptr(), t["cursor"].data_ptr(),
                                             t["tile_expert"].data_ptr(), t["n_tiles"].data_ptr(), t["slot_row"].data_ptr(), max_rows,
                                             t["pos"].data_ptr(), torch.cuda.current_stream(dev).cuda_stream))
        return t

    def _tensor_core_ok(self, h, slots):
        W = h.shape[1]
        return (self.dtype == torch.bfloat16 and h.dtype == torch.bfloat16 and h.is_contiguous() and W % 64 == 0 and self.F % 64 == 0
                and slots >= self.tc_min_rows_per_expert * self.E and bool(_core_lib()))

    def _forward_tensor_core(self, h, ids, slots):
        """Long bfloat16 steps: rows gathered into the binned order (runs padded to the 128-row tiles of the tcgen05 GEMM), then ONE
        grouped GEMM per projection: every row tile multiplies its expert's matrix, picked from the device-side tile table, and only
        the tiles that exist are computed — no host round trip."""
        from . import capi
        core, E, top, W, F, dev = _core_lib(), self.E, self.top, h.shape[1], self.F, h.device
        s = torch.cuda.current_stream(dev).cuda_stream
        t = self._bin(ids, slots, 128)
        rows, di = t["max_rows"], dev.index or 0
        src = torch.div(t["slot_row"].clamp_min(0), top, rounding_mode="floor").to(torch.int64)     # padding rows read token 0; never used
        xs = h.index_select(0, src)
        F1 = self.w_gu.shape[1]
        gu = torch.empty((rows, F1), dtype=torch.bfloat16, device=dev)
        capi.check(core.kb2_linear_bf16_grouped(xs.data_ptr(), self.w_gu.data_ptr(), gu.data_ptr(), rows, F1, W, 0, t["tile_expert"].data_ptr(),
                                                t["n_tiles"].data_ptr(), E, di, s))
        act = ops.glu(gu, torch.bfloat16, self.act_kind, n_tiles=t["n_tiles"], tile_rows=128)
        y = torch.empty((rows, W), dtype=torch.float32, device=dev)
        capi.check(core.kb2_linear_bf16_grouped(act.data_ptr(), self.w_down.data_ptr(), y.data_ptr(), rows, W, F, 1, t["tile_expert"].data_ptr(),
                                                t["n_tiles"].data_ptr(), E, di, s))
        return y, t["pos"]

    def route(self, h: torch.Tensor):
        """(ids, weights, router product [T, >= E + identity] whose column sg_col is the shared expert's gate input)."""
        z = lin(h, self.w_router, torch.float32, min_n=16)
        return ops.route(z, self.correction, self.top, self.groups, self.keep, self.score, self.renorm, self.out_scale, self.group_score,
                         experts=self.E + self.ident) + (z,)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        lib, T, W, E, top = ops.load(), h.shape[0], h.shape[1], self.E, self.top
        dev, s = h.device, torch.cuda.current_stream(h.device).cuda_stream
        ids, wts, z = self.route(h)
        dt, dtc = self.dtype, ops.dt_code(self.dtype)
        slots = T * top
        y = pos = None
        if E and T <= self.gemv_max_tokens:
            F2 = self.w_gu.shape[1]
            gu = torch.empty((slots, F2), dtype=dt, device=dev)
            ops.check(lib.kb2_seq_moe_gemv(h.data_ptr(), ops.dt_code(h.dtype), h.stride(0), top, ids.data_ptr(), E, self.w_gu.data_ptr(), dtc, W,
                                           F2 * W, gu.data_ptr(), dtc, F2, slots, F2, W, s))
            act = ops.glu(gu, dt, self.act_kind)
            y = torch.empty((slots, W), dtype=torch.float32, device=dev)
            ops.check(lib.kb2_seq_moe_gemv(act.data_ptr(), dtc, self.F, 1, ids.data_ptr(), E, self.w_down.data_ptr(), dtc, self.F, W * self.F,
                                           y.data_ptr(), 0, W, slots, W, self.F, s))
        elif E and self._tensor_core_ok(h, slots):
            y, pos = self._forward_tensor_core(h, ids, slots)
        elif E:
            F2, tile = self.w_gu.shape[1], self.tile
            t = self._bin(ids, slots, tile)
            max_rows, max_tiles, n_tiles, tile_expert, slot_row, pos = t["max_rows"], t["max_tiles"], t["n_tiles"], t["tile_expert"], t["slot_row"], t["pos"]
            gu = torch.empty((max_rows, F2), dtype=dt, device=dev)
            ops.check(lib.kb2_seq_moe_gemm(h.data_ptr(), ops.dt_code(h.dtype), h.stride(0), slot_row.data_ptr(), top, self.w_gu.data_ptr(), dtc, W,
                                           F2 * W, gu.data_ptr(), dtc, F2, F2, W, tile_expert.data_ptr(), n_tiles.data_ptr(), max_tiles, tile, s))
            act = ops.glu(gu, dt, self.act_kind, n_tiles=n_tiles, tile_rows=tile)
            y = torch.empty((max_rows, W), dtype=torch.float32, device=dev)
            ops.check(lib.kb2_seq_moe_gemm(act.data_ptr(), dtc, self.F, None, 1, self.w_down.data_ptr(), dtc, self.F, W * self.F, y.data_ptr(), 0,
                                           W, W, self.F, tile_expert.data_ptr(), n_tiles.data_ptr(), max_tiles, tile, s))
        shared = self.shared.forward(h) if self.shared is not None else None
        out = torch.empty((T, W), dtype=torch.float32, device=dev)
        sg = z[:, self.sg_col:] if (self.sg_col >= 0 and shared is not None) else None
        ops.check(lib.kb2_seq_moe_combine(ops._ptr(y), ops._ptr(pos), ids.data_ptr(), wts.data_ptr(), T, top, E, self.ident, h.data_ptr(),
                                          ops.dt_code(h.dtype), ops._ptr(shared), out.data_ptr(), W, ops._ptr(sg), z.stride(0), s))
        return out


class TokenSideInput:
    """weights: gate [dim, W], proj [W, dim], norm [W]; `table` [vocab, layers * dim] is shared by the layers, this one reads the
    columns [col0, col0 + dim).  forward returns y = proj(gelu(gate x) * table[token]); the caller adds rms_norm(y) * norm."""

    def __init__(self, weights: dict, table: torch.Tensor, col0: int, dim: int, dtype, device):
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        self.w_gate, self.w_proj = d(weights["gate"]), d(weights["proj"])
        self.norm = weights["norm"].to(device=device, dtype=torch.float32).contiguous()
        self.table, self.col0, self.dim, self.dtype = table, col0, dim, dtype

    def forward(self, x: torch.Tensor, tb: ops.StepTables) -> torch.Tensor:
        # x is the fp32 residual stream itself; a long bfloat16 step rounds it once so that the projection runs on the tensor cores
        a = x.to(torch.bfloat16) if (self.dtype == torch.bfloat16 and x.shape[0] >= 256 and _core_lib()) else x
        g = lin(a, self.w_gate, torch.float32)
        return lin(ops.side_gate(g, self.table, tb.tokens, self.col0, self.dtype), self.w_proj, torch.float32)
