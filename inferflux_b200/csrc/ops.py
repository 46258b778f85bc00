"""The kernel table of the product path: every operation of a step as a call into
the hand-written sm_100a library (plus cuBLAS for the bfloat16 matrix products,
where the reference uses it too).

There is no CPU path and no library model code here: making a `CudaKernels`
without a CUDA device, or without being able to build or load the library, raises.
Tensors are passed as raw device pointers on torch's current stream.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import BuildError, load_library

_DT = {torch.float32: 0, torch.bfloat16: 1}

_ERRORS = {-1: "a size or option the kernel does not take", -2: "unknown dtype",
           -3: "a pointer or stride breaks an alignment rule", -4: "a size beyond the kernel's stated maximum"}


class KernelError(RuntimeError):
    pass


class ScaledRows:
    """Rows of a norm without its row scale: `pre` = x * w in the run's dtype and `sumsq`
    [rows, chunks] float32, the chunks' sums of x^2.  The true rows are
    pre * rsqrt(sum(sumsq[row]) / hidden + eps); a matrix product that takes them applies that
    per-row factor to its accumulator.  `CudaKernels.materialize_rows` gives the plain tensor."""

    def __init__(self, pre: torch.Tensor, sumsq: torch.Tensor, eps: float):
        self.pre, self.sumsq, self.eps = pre, sumsq, float(eps)

    @property
    def shape(self):
        return self.pre.shape

    @property
    def dtype(self):
        return self.pre.dtype


class PartialSum:
    """The result of a matrix product whose K range was split over thread blocks:
    float32 partial sums [splits, rows, cols] that the consuming kernel adds, in split
    order, in the same pass in which it does its own work (residual add and norm, bias
    and rotation).  `CudaKernels.materialize` gives the plain tensor."""

    def __init__(self, parts: torch.Tensor, dtype: torch.dtype):
        self.parts = parts
        self.dtype = dtype                       # the dtype the sum stands for

    @property
    def shape(self):
        return self.parts.shape[1:]

    @property
    def splits(self) -> int:
        return self.parts.shape[0]


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# The current stream's handle of the current device, asked for at every launch: torch's own accessors
# when they are there (plain integers, a fraction of a microsecond), else through the Stream object
# (several microseconds).
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _RAW_STREAM is not None and _RAW_DEVICE is not None:
        return ctypes.c_void_p(_RAW_STREAM(_RAW_DEVICE()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise KernelError(f"{what}: refused ({_ERRORS.get(rc, rc)})")
    if rc >= 1000:
        raise KernelError(f"{what}: cuBLAS status {rc - 1000}")
    raise KernelError(f"{what}: CUDA error {rc}")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


_I, _F, _P, _LL = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong


class TurnedQueries:
    """Query rows [T, heads (dim + rot)] whose turned parts already lie in `latent`, the rows of queries in latent
    space [T, heads (rank + rot)] that the tiled latent attention reads."""
    __slots__ = ("rows", "latent")

    def __init__(self, rows, latent):
        self.rows, self.latent = rows, latent


class _StepArgs(ctypes.Structure):
    """IfxStepArgs of csrc/layer_forward.cu: one step's batch, the same for every layer."""
    _fields_ = ([(n, _I) for n in ("T", "num_decode", "num_tiles", "max_kv_len")]
                + [(n, _P) for n in ("positions", "token_req", "req_slot", "decode_rows", "decode_meta", "prefill_tiles",
                                     "norm_sumsq", "norm_tickets", "error_flag")]
                + [(n, _I) for n in ("skinny_max_rows", "swiglu_tiles", "swiglu_tiles_max_k", "tensor_core_prefill",
                                     "overlap_attention", "pad0")])


class _LayerArgs(ctypes.Structure):
    """IfxLayerArgs: one layer's sizes, constants, weights and cache."""
    _fields_ = ([(n, _I) for n in ("hidden", "inter", "nq", "nkv", "d", "window", "rot", "interleaved")]
                + [(n, _F) for n in ("scale", "eps_in", "eps_post")] + [("write_cache", _I)]
                + [(n, _P) for n in ("norm_in_w", "norm_post_w", "b_qkv", "inv_freq", "w_qkv", "w_o", "w_gate_up", "w_down",
                                     "kv_pool", "block_table")]
                + [(n, _I) for n in ("max_blocks", "page_size", "num_pages", "pad0")])


class _LayerIO(ctypes.Structure):
    """IfxLayerIO: what changes from call to call, and what comes back."""
    _fields_ = [("x", _P), ("pending_tensor", _P), ("pending_parts", _P), ("pending_splits", _I), ("parity", _I),
                ("ws", _P), ("ws_bytes", _LL), ("out_tensor", _P), ("out_parts", _P), ("out_splits", _I),
                ("launches", _I), ("library_calls", _I), ("pad0", _I)]


class CudaKernels:
    """Kernel table on one CUDA device."""

    name = "cuda-sm100a"
    fuses_single_token_conv = True     # postnorm_add takes a short convolution for steps of single tokens

    def __init__(self, device="cuda"):
        if not torch.cuda.is_available():
            raise BuildError("no CUDA device: the engine has no CPU path")
        self.device = torch.device(device)
        self.lib = load_library()
        for fn in ("ifx_embed", "ifx_rmsnorm", "ifx_silu_mul", "ifx_residual_add", "ifx_gather_rows",
                   "ifx_scatter_i32", "ifx_rope_append", "ifx_attention_generic", "ifx_gemm_generic",
                   "ifx_gemm_cublas_bf16", "ifx_cublas_init", "ifx_argmax", "ifx_penalties", "ifx_logit_bias",
                   "ifx_sample", "ifx_sample_blocks", "ifx_attention_mma_supports", "ifx_attention_prefill_bf16",
                   "ifx_attention_prefill_tcgen05", "ifx_attention_prefill_tcgen05_supports", "ifx_attention_decode_max_splits",
                   "ifx_attention_decode_bf16", "ifx_gemm_skinny", "ifx_residual_add_partial",
                   "ifx_reduce_partial", "ifx_reduce_add_rmsnorm", "ifx_argmax_chunks", "ifx_relay_i32", "ifx_prenorm", "ifx_scale_rows",
                   "ifx_gemm_tcgen05", "ifx_postnorm_add_rmsnorm", "ifx_concat_cast", "ifx_xielu", "ifx_softcap",
                   "ifx_short_conv", "ifx_latent_norm_append", "ifx_latent_attention_generic", "ifx_latent_attention_mma",
                   "ifx_latent_attention_mma_supports", "ifx_gemm_cublas_bf16_batched", "ifx_gemm_skinny_act",
                   "ifx_attention_generic_ex", "ifx_norm_rope_append", "ifx_token_shift_mix", "ifx_cast_rows",
                   "ifx_wkv_scan", "ifx_moe_route", "ifx_moe_experts", "ifx_tanh_rows",
                   "ifx_attention_prefill_bf16_ex", "ifx_attention_decode_bf16_ex", "ifx_moe_sorted_rows", "ifx_moe_sort",
                   "ifx_moe_gather", "ifx_moe_combine", "ifx_gemm_tcgen05_grouped", "ifx_attention_prefill_tcgen05_ex",
                   "ifx_groupnorm_stream", "ifx_residual_add_scaled", "ifx_gelu_mul_table", "ifx_embed_scaled", "ifx_scale_f32",
                   "ifx_delta_rule_scan", "ifx_latent_rope_append", "ifx_latent_attention_generic_rot", "ifx_moe_route_ex",
                   "ifx_moe_experts_ex", "ifx_gemm_tcgen05_grouped_glu", "ifx_latent_attention_mma_rot", "ifx_latent_attention_mma_supports_rot",
                   "ifx_moe_route_kind", "ifx_moe_experts_glu", "ifx_gemm_tcgen05_grouped_glu_offset", "ifx_norm_rope_append_ex",
                   "ifx_attention_generic_sink", "ifx_short_conv_ex", "ifx_decay_scan", "ifx_decay_scan_split", "ifx_bigram_add",
                   "ifx_rmsnorm_pair", "ifx_gate_mul", "ifx_gated_groupnorm", "ifx_pair_combine", "ifx_residual_add_vectors",
                   "ifx_attention_prefill_tcgen05_sink", "ifx_attention_prefill_bf16_sink", "ifx_attention_decode_bf16_sink"):
            getattr(self.lib, fn).restype = ctypes.c_int
        self.lib.ifx_delta_rule_scratch_floats.restype = ctypes.c_longlong
        self.lib.ifx_sample_scratch_bytes.restype = ctypes.c_longlong
        self.lib.ifx_latent_attention_mma_workspace.restype = ctypes.c_longlong
        # latent attention on the tensor-core tiles (0: the per-token kernel, for comparisons)
        self.latent_tiles = os.environ.get("INFERFLUX_B200_LATENT_TILES", "1") != "0"
        with torch.cuda.device(self.device):
            _check(self.lib.ifx_cublas_init(), "cublas init")
        if os.environ.get("INFERFLUX_B200_CARVEOUT", "") != "":    # for measurements: -1 leaves the split to the driver
            self.lib.ifx_set_shared_carveout(int(os.environ["INFERFLUX_B200_CARVEOUT"]))
        if os.environ.get("INFERFLUX_B200_PDL", "1") == "0":      # for measurements: no overlap of consecutive kernels
            self.lib.ifx_set_pdl(0)
        # prompt portions on the tcgen05 attention kernel (0: the mma.sync kernel, for comparisons)
        self.tensor_core_prefill = os.environ.get("INFERFLUX_B200_TCGEN05_ATTENTION", "1") != "0"
        # gate/up of prompt portions on the own tcgen05 tiles with the activation fused (0: cuBLAS + silu kernel)
        self.swiglu_tiles = os.environ.get("INFERFLUX_B200_SWIGLU_TILES", "1") != "0"
        self.launches = 0            # kernels of this library launched so far
        self.library_calls = 0       # cuBLAS products called so far
        # scratch of the many-block reduce + norm: sums of squares per (row, chunk), a ticket per row
        self._norm_sumsq = torch.zeros(128 * 64, dtype=torch.float32, device=self.device)
        self._norm_tickets = torch.zeros(128, dtype=torch.int32, device=self.device)
        self._sample_scratch, self._sample_capacity = None, 0   # zeroed once; the sampling kernels leave it zero
        self._argmax_val = torch.zeros(256 * 32, dtype=torch.float32, device=self.device)
        self._argmax_idx = torch.zeros(256 * 32, dtype=torch.int32, device=self.device)
        self._argmax_tickets = torch.zeros(256, dtype=torch.int32, device=self.device)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)   # set by a kernel whose bounded wait ran out
        # whole layers from native code (0: every part launches its kernels from Python, the general way)
        self.native_layers = os.environ.get("INFERFLUX_B200_NATIVE_LAYER", "1") != "0"
        # in a natively run layer of a mixed step, the two attention kernels side by side on two streams
        self.overlap_attention = os.environ.get("INFERFLUX_B200_ATTENTION_OVERLAP", "1") != "0"
        self.lib.ifx_layer_forward.restype = ctypes.c_int
        self.lib.ifx_layer_workspace_bytes.restype = ctypes.c_longlong
        self._layer_ws, self._layer_ws_all, self._layer_views = None, [], {}
        self._layer_io = _LayerIO()
        self._layer_io_ref = ctypes.byref(self._layer_io)
        self._layer_parity = 0
        self.native_layer_calls = 0

    # ------------------------------------------------------------- elementwise
    def embed(self, table, token_ids, vocab, scale=1.0):
        T, H = token_ids.numel(), table.shape[1]
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
        if scale != 1.0:
            _check(self.lib.ifx_embed_scaled(_ptr(table), _ptr(token_ids), _ptr(out), T, H, int(vocab), ctypes.c_float(scale),
                                             _DT[table.dtype], _stream()), "embed")
            self.launches += 1
            return out
        _check(self.lib.ifx_embed(_ptr(table), _ptr(token_ids), _ptr(out), T, H, int(vocab), _DT[table.dtype],
                                  _stream()), "embed")
        self.launches += 1
        return out

    def rmsnorm(self, x, w, eps, out_dtype, groups=1):
        _need(x.dtype == torch.float32 and w.dtype == torch.float32, "rmsnorm: x and w must be float32")
        T, H = x.shape
        out = torch.empty((T, H), dtype=out_dtype, device=x.device)
        if groups > 1:
            _need(x.is_contiguous() and H % groups == 0, "rmsnorm: the groups must cut a contiguous row evenly")
            _check(self.lib.ifx_groupnorm_stream(
                _ptr(x), _ptr(None), _ptr(None), ctypes.c_float(0.0), _ptr(w), ctypes.c_float(eps), int(groups), _ptr(out),
                _ptr(None), T, H, 0, _DT[out_dtype], 1, _ptr(None), 0, _ptr(None), ctypes.c_longlong(0), _ptr(None),
                _ptr(None), _stream()), "rmsnorm (groups)")
            self.launches += 1
            return out
        _check(self.lib.ifx_rmsnorm(_ptr(x), _ptr(None), _ptr(w), _ptr(out), T, H, ctypes.c_float(eps), 0,
                                    _DT[out_dtype], _stream()), "rmsnorm")
        self.launches += 1
        return out

    def add_rmsnorm(self, x, delta, w, eps, out_dtype):
        """x += delta (in place), then the norm of the sum.  `delta` is a tensor in the run's
        dtype or a PartialSum, whose slices are added in the same pass."""
        _need(x.dtype == torch.float32 and w.dtype == torch.float32, "add_rmsnorm: x and w must be float32")
        T, H = x.shape
        out = torch.empty((T, H), dtype=out_dtype, device=x.device)
        if isinstance(delta, PartialSum):
            _need(tuple(delta.shape) == (T, H), "add_rmsnorm: partial sums do not match x")
            chunks = -(-H // 512)
            if T <= self._norm_tickets.numel() and T * chunks <= self._norm_sumsq.numel():
                _check(self.lib.ifx_reduce_add_rmsnorm(
                    _ptr(x), _ptr(delta.parts), _ptr(w), _ptr(out), T, H, ctypes.c_float(eps), delta.splits,
                    _ptr(self._norm_sumsq), _ptr(self._norm_tickets), _DT[out_dtype], _stream()), "reduce_add_rmsnorm")
                self.launches += 1
                return out
            src, splits = delta.parts, delta.splits
        else:
            _need(delta.dtype == out_dtype and delta.shape == x.shape, "add_rmsnorm: delta must match x and the dtype")
            src, splits = delta, 0
        _check(self.lib.ifx_rmsnorm(_ptr(x), _ptr(src), _ptr(w), _ptr(out), T, H, ctypes.c_float(eps), splits,
                                    _DT[out_dtype], _stream()), "add_rmsnorm")
        self.launches += 1
        return out

    def prenorm(self, x, delta, w, eps, out_dtype):
        """The norm for a consumer that takes ScaledRows (x += delta first, as add_rmsnorm).
        Few bfloat16 rows: one pass that leaves x * w and per-chunk sums of squares, the row scale
        being applied by the matrix product that follows.  Otherwise the plain normed tensor."""
        T, H = x.shape
        if out_dtype != torch.bfloat16 or T > self.SKINNY_MAX_ROWS or H % 8:
            return self.rmsnorm(x, w, eps, out_dtype) if delta is None else self.add_rmsnorm(x, delta, w, eps, out_dtype)
        pre = torch.empty((T, H), dtype=out_dtype, device=x.device)
        sumsq = torch.empty((T, -(-H // 512)), dtype=torch.float32, device=x.device)
        if isinstance(delta, PartialSum):
            _need(tuple(delta.shape) == (T, H), "prenorm: partial sums do not match x")
            src, splits = delta.parts, delta.splits
        else:
            _need(delta is None or (delta.dtype == out_dtype and delta.shape == x.shape), "prenorm: delta must match x")
            src, splits = delta, 0
        _check(self.lib.ifx_prenorm(_ptr(x), _ptr(src), _ptr(w), _ptr(pre), _ptr(sumsq), T, H, splits, _DT[out_dtype],
                                    _stream()), "prenorm")
        self.launches += 1
        return ScaledRows(pre, sumsq, eps)

    def materialize_rows(self, h):
        """A plain tensor from what `prenorm` returned."""
        if not isinstance(h, ScaledRows):
            return h
        T, H = h.shape
        out = torch.empty((T, H), dtype=h.dtype, device=h.pre.device)
        _check(self.lib.ifx_scale_rows(_ptr(h.pre), _ptr(h.sumsq), _ptr(out), T, H, ctypes.c_float(h.eps),
                                       _DT[h.dtype], _stream()), "scale_rows")
        self.launches += 1
        return out

    def residual_add(self, x, delta):
        T, H = x.shape
        if isinstance(delta, PartialSum):
            _check(self.lib.ifx_residual_add_partial(_ptr(x), _ptr(delta.parts), T, H, delta.splits, _stream()),
                   "residual_add")
        else:
            _check(self.lib.ifx_residual_add(_ptr(x), _ptr(delta), T, H, _DT[delta.dtype], _stream()), "residual_add")
        self.launches += 1

    def materialize(self, value, bias=None):
        """A plain tensor from what `linear(..., allow_partial=True)` returned."""
        if not isinstance(value, PartialSum):
            return value if bias is None else value + bias.to(value.dtype)
        T, N = value.shape
        out = torch.empty((T, N), dtype=value.dtype, device=value.parts.device)
        _check(self.lib.ifx_reduce_partial(_ptr(value.parts), _ptr(bias), _ptr(out), T, N, value.splits,
                                           _DT[value.dtype], _stream()), "reduce_partial")
        self.launches += 1
        return out

    def silu_mul(self, gate_up):
        T, two_i = gate_up.shape
        out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
        _check(self.lib.ifx_silu_mul(_ptr(gate_up), _ptr(out), T, two_i // 2, _DT[gate_up.dtype], _stream()),
               "silu_mul")
        self.launches += 1
        return out

    def gather_rows(self, x, rows):
        R, H = rows.numel(), x.shape[1]
        out = torch.empty((R, H), dtype=torch.float32, device=x.device)
        _check(self.lib.ifx_gather_rows(_ptr(x), _ptr(rows), _ptr(out), R, H, x.shape[0], _stream()), "gather_rows")
        self.launches += 1
        return out

    def scatter_i32(self, table, index, value):
        n = index.numel()
        if n:
            _check(self.lib.ifx_scatter_i32(_ptr(table), _ptr(index), _ptr(value), n, table.numel(), _stream()),
                   "scatter_i32")
            self.launches += 1

    def relay_i32(self, dst, dst_index, src, src_index):
        n = dst_index.numel()
        if n:
            _check(self.lib.ifx_relay_i32(_ptr(dst), _ptr(dst_index), _ptr(src), _ptr(src_index), n, dst.numel(),
                                          src.numel(), _stream()), "relay_i32")
            self.launches += 1

    # ------------------------------------------------------------------ linear
    # The weight-streaming kernel takes up to 256 rows; in a whole step it beats cuBLAS up to about 160
    # (measured at the 7B shape: 4.5 against 4.9 ms at 129 rows, 5.2 against 5.0 ms at 192).
    SKINNY_MAX_ROWS = 160

    def linear(self, a, w, bias=None, out_dtype=None, allow_partial=False):
        """out[T, N] = a[T, K] . w[N, K]^T (+ bias), float32 accumulation.  float32 runs use
        the CUDA-core product.  bfloat16 runs with up to 256 rows use the tcgen05 weight-streaming
        kernel; with `allow_partial` a narrow product is split over K and comes back as a
        PartialSum for a consumer that adds the slices itself.  More rows go to cuBLAS."""
        rows = a if isinstance(a, ScaledRows) else None
        if rows is not None:
            a = rows.pre
        _need(a.dtype == w.dtype, f"linear: activations are {a.dtype}, weights {w.dtype}")
        _need(a.is_contiguous() and w.is_contiguous(), "linear: operands must be contiguous")
        T, K = a.shape
        N = w.shape[0]
        _need(w.shape[1] == K, f"linear: inner sizes differ ({K} vs {w.shape[1]})")
        out_dtype = out_dtype or a.dtype
        if T == 0:
            return torch.empty((T, N), dtype=out_dtype, device=a.device)
        if rows is not None and not (T <= self.SKINNY_MAX_ROWS and K % 8 == 0 and w.data_ptr() % 16 == 0):
            a, rows = self.materialize_rows(rows), None
        if a.dtype == torch.float32:
            _need(out_dtype == torch.float32, "linear: a float32 product gives float32")
            out = torch.empty((T, N), dtype=out_dtype, device=a.device)
            _check(self.lib.ifx_gemm_generic(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), T, N, K, 0, 0, _stream()),
                   "gemm (float32)")
            self.launches += 1
            return out
        if T <= self.SKINNY_MAX_ROWS and K % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
            tiles = -(-N // 128)
            kblocks = -(-K // 64)
            # up to 128 rows: two blocks a SM and up to 10 K slices; above, a block owns its SM (32 KB of
            # activations a stage) and every slice costs a [T, N] float32 round trip: at most 5
            slots, most = (296, 10) if T <= 128 else (148, 5)
            splits = max(1, min(slots // tiles, most, kblocks // 4)) if allow_partial and bias is None else 1
            if splits > 1:
                parts = self.linear_skinny(a, w, None, splits=splits, mode=1, rows=rows)
                return PartialSum(parts, out_dtype)
            if tiles >= 74 or allow_partial or rows is not None:
                return self.linear_skinny(a, w, bias, out_dtype=out_dtype, splits=1, mode=0, rows=rows)
        out = torch.empty((T, N), dtype=out_dtype, device=a.device)
        _check(self.lib.ifx_gemm_cublas_bf16(_ptr(a), _ptr(w), _ptr(out), T, N, K, _DT[out_dtype], _stream()),
               "gemm (bfloat16)")
        self.library_calls += 1
        if bias is not None:
            out += bias.to(out.dtype)
        return out

    # The many-rows tcgen05 product with SiLU(gate)*up in its epilogue against cuBLAS followed by the activation
    # kernel, measured on a B200 (us a layer, 256 / 512 / 2,048 rows): Qwen2.5-1.5B sizes 21 vs 27, 31 vs 37, 94 vs 110;
    # 7B sizes 63 vs 79, 107 vs 107, 373 vs 381; 32B sizes (inner size 5120) 126 vs 136, 217 vs 212, 851 vs 779.
    # So it is used up to an inner size of 4096.
    SWIGLU_TILES_MAX_K = 4096

    def linear_swiglu(self, a, w_gate_up):
        """silu(a . Wg^T) * (a . Wu^T) with Wg and Wu stacked in w_gate_up [2 I, K]: one kernel
        with both accumulators for few rows, else the product followed by the activation kernel."""
        rows = a if isinstance(a, ScaledRows) else None
        if rows is not None:
            a = rows.pre
        T, K = a.shape
        inter = w_gate_up.shape[0] // 2
        if (a.dtype == torch.bfloat16 and 0 < T <= self.SKINNY_MAX_ROWS and K % 8 == 0 and a.data_ptr() % 16 == 0
                and w_gate_up.data_ptr() % 16 == 0):
            return self.linear_skinny(a, w_gate_up, None, splits=1, mode=2, n_out=inter, up_row_offset=inter, rows=rows)
        if rows is not None:
            a = self.materialize_rows(rows)
        if (self.swiglu_tiles and a.dtype == torch.bfloat16 and K % 8 == 0 and K <= self.SWIGLU_TILES_MAX_K
                and a.data_ptr() % 16 == 0 and w_gate_up.data_ptr() % 16 == 0 and a.is_contiguous()):
            return self.linear_tiles(a, w_gate_up, swiglu=True)        # many rows: own tcgen05 tiles, activation fused
        return self.silu_mul(self.linear(a, w_gate_up))

    def linear_xielu(self, a, w, a_pos, a_neg):
        """xielu(a . w^T): for few bfloat16 rows and a product wide enough to fill the SMs without K slices, the
        weight-streaming kernel with the activation on its result; otherwise the product (maybe in K slices)
        followed by the activation kernel, which adds the slices."""
        T, K = a.shape
        N = w.shape[0]
        if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < T <= self.SKINNY_MAX_ROWS and K % 8 == 0
                and a.is_contiguous() and w.is_contiguous() and w.shape[1] == K and a.data_ptr() % 16 == 0
                and w.data_ptr() % 16 == 0 and -(-N // 128) >= 74):
            out = torch.empty((T, N), dtype=torch.bfloat16, device=a.device)
            _check(self.lib.ifx_gemm_skinny_act(_ptr(a), _ptr(w), _ptr(None), _ptr(out), T, N, K, w.shape[0], 0, _ptr(None), 0,
                                                ctypes.c_float(0.0), 1, ctypes.c_float(a_pos), ctypes.c_float(a_neg),
                                                _ptr(self.error_flag), _stream()), "gemm_skinny (xielu)")
            self.launches += 1
            return out
        return self.xielu(self.linear(a, w, allow_partial=True), a_pos, a_neg)

    def check_errors(self):
        """Raise if a kernel reported that one of its bounded waits ran out (reads the device flag)."""
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            raise KernelError(f"a kernel gave up waiting on a barrier (code {code}); its output is not valid")

    def linear_skinny(self, a, w, bias=None, out_dtype=None, splits=1, mode=0, n_out=None, up_row_offset=0, rows=None):
        """The tcgen05 weight-streaming product for up to 256 token rows.
        mode 0: out[T, N] (+bias); mode 1: float32 partial sums [splits, T, N]; mode 2: silu(gate) * up.
        `rows`: the ScaledRows whose `pre` is `a`; the product then applies their row scale."""
        T, K = a.shape
        N = n_out if n_out is not None else w.shape[0]
        _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear_skinny: bfloat16 only")
        _need(a.is_contiguous() and w.is_contiguous() and w.shape[1] == K, "linear_skinny: bad operands")
        out_dtype = out_dtype or torch.bfloat16
        out = partials = None
        if mode == 1:
            partials = torch.empty((splits, T, N), dtype=torch.float32, device=a.device)
        else:
            out = torch.empty((T, N), dtype=out_dtype, device=a.device)
        _check(self.lib.ifx_gemm_skinny(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), _ptr(partials), T, N, K, w.shape[0],
                                        splits, mode, up_row_offset, int(out_dtype == torch.float32),
                                        _ptr(None if rows is None else rows.sumsq),
                                        0 if rows is None else rows.sumsq.shape[1],
                                        ctypes.c_float(0.0 if rows is None else rows.eps),
                                        _ptr(self.error_flag), _stream()), "gemm_skinny")
        self.launches += 1
        return partials if mode == 1 else out

    def linear_tiles(self, a, w, swiglu=False):
        """The many-rows tcgen05 product (csrc/gemm_tcgen05.cu): a . w^T in bfloat16, or, with `swiglu`,
        silu(a . Wg^T) * (a . Wu^T) for w = [Wg; Wu] stacked, without the [T, 2 I] round trip."""
        T, K = a.shape
        _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear_tiles: bfloat16 only")
        _need(a.is_contiguous() and w.is_contiguous() and w.shape[1] == K and K % 8 == 0, "linear_tiles: bad operands")
        N = w.shape[0] // 2 if swiglu else w.shape[0]
        out = torch.empty((T, N), dtype=torch.bfloat16, device=a.device)
        _check(self.lib.ifx_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(out), T, N, K, w.shape[0], int(bool(swiglu)),
                                         N if swiglu else 0, _ptr(self.error_flag), _stream()), "gemm_tcgen05")
        self.launches += 1
        return out

    def linear_generic(self, a, w, bias=None, out_dtype=None):
        """The CUDA-core product for any dtype (used by tests and as the refusal-free path)."""
        T, K = a.shape
        N = w.shape[0]
        out_dtype = out_dtype or a.dtype
        out = torch.empty((T, N), dtype=out_dtype, device=a.device)
        _check(self.lib.ifx_gemm_generic(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), T, N, K, _DT[a.dtype],
                                         _DT[out_dtype], _stream()), "gemm_generic")
        self.launches += 1
        return out

    # ------------------------------------------------------------ whole layers
    def _native_parts(self, block):
        """The block's (mixer, ffn, norm before the mixer, norm before the ffn) if it is exactly the arrangement
        and the parts that csrc/layer_forward.cu runs (no subclass: one may have changed a forward), else None."""
        known = getattr(block, "_native_parts", False)
        if known is not False:
            return known
        from ..parts.attention import Attention
        from ..parts.block import PreNormBlock
        from ..parts.mlp import SwiGLU
        from ..parts.norm import RMSNorm
        parts = None
        if type(block) is PreNormBlock:
            m, f, n1, n2 = block.mixer, block.ffn, block.norm_mixer, block.norm_ffn
            if (type(m) is Attention and not m.general and type(f) is SwiGLU and type(n1) is RMSNorm and type(n2) is RMSNorm
                    and m.hidden == f.hidden == n1.size == n2.size):
                parts = (m, f, n1, n2)
        block._native_parts = parts
        block._native_layers = {}
        return parts

    def _native_workspace(self, T, parts):
        m, f = parts[0], parts[1]
        need = int(self.lib.ifx_layer_workspace_bytes(T, m.hidden, m.nq * m.d, m.nkv * m.d, f.inter, self.SKINNY_MAX_ROWS))
        ws = self._layer_ws
        if ws is None or ws.numel() < need:
            if torch.cuda.is_current_stream_capturing():
                return None                              # no allocation inside a graph: the parts run one by one
            # graphs captured earlier hold the old one's address: it stays alive
            ws = torch.empty(max(need, 2 * (0 if ws is None else ws.numel())), dtype=torch.uint8, device=self.device)
            self._layer_ws_all.append(ws)
            self._layer_ws = ws
            self._layer_views = {}
        return ws

    def _native_layer_args(self, block, parts, ctx, cache):
        """The C structure of one layer with one cache (sizes, constants, weight and cache addresses), made when
        the pair first runs and kept on the block; None if the cache or the weights are not bfloat16."""
        m, f, n1, n2 = parts
        tensors = (m.w_qkv, m.w_o, m.b_qkv, f.w_gate_up, f.w_down, n1.weight, n2.weight)
        kv, table = cache.kv, cache.block_table
        kv_ptr = kv.data_ptr()
        # everything of the cache that the structure holds: another runner may get the same addresses
        key = (kv_ptr, table.data_ptr(), cache.writes, cache.page_size, table.shape[1], kv.shape[0])
        entry = block._native_layers.get(key)
        if entry is None or any(a is not b for a, b in zip(entry[1], tensors)):
            if kv.dtype is not torch.bfloat16 or m.w_qkv.dtype is not torch.bfloat16:
                return None
            rotary = m.position.rotary(ctx.device) if m.position is not None else None
            la = _LayerArgs(
                hidden=m.hidden, inter=f.inter, nq=m.nq, nkv=m.nkv, d=m.d, window=int(m.window or 0),
                rot=0 if rotary is None else int(rotary.rotary_dim),
                interleaved=int(bool(rotary.interleaved)) if rotary is not None else 0,
                scale=m.scale, eps_in=n1.eps, eps_post=n2.eps, write_cache=int(bool(cache.writes)),
                norm_in_w=n1.weight.data_ptr(), norm_post_w=n2.weight.data_ptr(),
                b_qkv=0 if m.b_qkv is None else m.b_qkv.data_ptr(),
                inv_freq=0 if rotary is None else rotary.inv_freq.data_ptr(),
                w_qkv=m.w_qkv.data_ptr(), w_o=m.w_o.data_ptr(), w_gate_up=f.w_gate_up.data_ptr(),
                w_down=f.w_down.data_ptr(), kv_pool=kv_ptr, block_table=table.data_ptr(),
                max_blocks=table.shape[1], page_size=cache.page_size, num_pages=kv.shape[0])
            entry = (la, tensors, rotary, table, ctypes.byref(la))      # the tensors stay alive with the addresses
            if len(block._native_layers) >= 8:           # caches come and go with their runners
                block._native_layers.clear()
            block._native_layers[key] = entry
        return entry[4]

    def _native_step_args(self, ctx, device):
        """The C structure of the step's batch (metadata addresses, counts, this table's knobs), made at the
        step's first layer and kept on the context."""
        step = getattr(ctx, "_native_step", None)
        if step is None or step[1] is not ctx.positions or step[0].max_kv_len != ctx.max_kv_len:
            if "attn.prefill_tiles" not in ctx.extra:      # a step context built without the mixer as a provider
                for name, vals in self.attention_sections(ctx).items():
                    ctx.extra[name] = torch.tensor(vals, dtype=torch.int32, device=device)
                    ctx.extra_len[name] = len(vals)
            sa = _StepArgs(
                T=ctx.num_tokens, num_decode=ctx.extra_len["attn.decode_rows"],
                num_tiles=ctx.extra_len["attn.prefill_tiles"] // 4,
                max_kv_len=int(ctx.max_kv_len), positions=ctx.positions.data_ptr(), token_req=ctx.token_req.data_ptr(),
                req_slot=ctx.req_slot.data_ptr(), decode_rows=ctx.extra["attn.decode_rows"].data_ptr(),
                decode_meta=ctx.extra["attn.decode_meta"].data_ptr(),
                prefill_tiles=ctx.extra["attn.prefill_tiles"].data_ptr(), norm_sumsq=self._norm_sumsq.data_ptr(),
                norm_tickets=self._norm_tickets.data_ptr(), error_flag=self.error_flag.data_ptr(),
                skinny_max_rows=self.SKINNY_MAX_ROWS, swiglu_tiles=int(self.swiglu_tiles),
                swiglu_tiles_max_k=self.SWIGLU_TILES_MAX_K, tensor_core_prefill=int(self.tensor_core_prefill),
                overlap_attention=int(self.overlap_attention))
            step = ctx._native_step = (sa, ctx.positions, ctypes.byref(sa))
        return step[2]

    def fused_prenorm_layer(self, block, x, pending, ctx, cache):
        """One native call for a pre-norm layer of attention and SwiGLU in bfloat16: the kernels that the parts
        would launch one by one, chosen by the same rules, launched from csrc/layer_forward.cu.  Returns
        (x, the layer's last delta, unadded) or None if this block, dtype or cache is not what that code runs."""
        if not self.native_layers or ctx.dtype is not torch.bfloat16 or cache.kv is None or cache.block_table is None:
            return None
        parts = self._native_parts(block)
        if parts is None or x.dtype is not torch.float32:
            return None
        m, f, n1, n2 = parts
        if block.mixer is not m or block.ffn is not f or block.norm_mixer is not n1 or block.norm_ffn is not n2:
            block._native_parts = False                  # a part was exchanged: look again
            return self.fused_prenorm_layer(block, x, pending, ctx, cache)
        T = ctx.num_tokens
        ws = self._native_workspace(T, parts)
        if ws is None:
            return None
        layer = self._native_layer_args(block, parts, ctx, cache)
        if layer is None:
            return None
        step = self._native_step_args(ctx, x.device)
        io = self._layer_io
        io.x = x.data_ptr()
        if pending is None:
            io.pending_tensor, io.pending_parts, io.pending_splits = 0, 0, 0
        elif isinstance(pending, PartialSum):
            if tuple(pending.shape) != tuple(x.shape):
                return None
            io.pending_tensor, io.pending_parts, io.pending_splits = 0, pending.parts.data_ptr(), pending.splits
        else:
            if pending.dtype is not torch.bfloat16 or pending.shape != x.shape or not pending.is_contiguous():
                return None
            io.pending_tensor, io.pending_parts, io.pending_splits = pending.data_ptr(), 0, 0
        parity = self._layer_parity = 1 - self._layer_parity
        io.parity = parity
        io.ws, io.ws_bytes = ws.data_ptr(), ws.numel()
        rc = self.lib.ifx_layer_forward(step, layer, self._layer_io_ref, _stream())
        self.launches += io.launches
        self.library_calls += io.library_calls
        self.native_layer_calls += 1
        _check(rc, "layer (native)")
        view = (T, m.hidden, parity, io.out_splits)
        out = self._layer_views.get(view)
        if out is None:
            at = (io.out_parts or io.out_tensor) - ws.data_ptr()
            if io.out_splits:
                n = io.out_splits * T * m.hidden * 4
                out = PartialSum(ws[at:at + n].view(torch.float32).view(io.out_splits, T, m.hidden), torch.bfloat16)
            else:
                out = ws[at:at + T * m.hidden * 2].view(torch.bfloat16).view(T, m.hidden)
            self._layer_views[view] = out
        return x, out

    # --------------------------------------------------------------- attention
    PREFILL_TILE = 256         # query rows per work item of the prompt-portion attention kernels

    def attention_sections(self, ctx):
        """Work lists of the attention kernels for one step, from the step's spans:
        attn.decode_rows[D] (flat indices of spans of one token), attn.decode_meta[D,4] (flat index,
        position, slot, 0: what the decode kernel needs of a token, in one 16-byte load),
        attn.prefill_tiles[P,4] (request, first flat row, rows, first position) for longer spans."""
        rows, meta, tiles, base = [], [], [], 0
        for r, ((start, n), slot) in enumerate(zip(ctx.spans, ctx.slots_host)):
            if n == 1:
                rows.append(base)
                meta.extend((base, start, int(slot), 0))
            else:
                for off in range(0, n, self.PREFILL_TILE):
                    tiles.extend((r, base + off, min(self.PREFILL_TILE, n - off), start + off))
            base += n
        return {"attn.decode_rows": rows, "attn.decode_meta": meta, "attn.prefill_tiles": tiles}

    @staticmethod
    def small_attention_grid(ctx, nkv):
        """1 if the step is decoded tokens only and their attention grid (tokens x kv heads x up to 8 key slices)
        leaves SMs free: the rotation kernel then lets it in early."""
        extra_len = getattr(ctx, "extra_len", None) or {}
        if "attn.decode_rows" not in extra_len:
            return 0
        return int(extra_len.get("attn.prefill_tiles", 0) == 0 and extra_len["attn.decode_rows"] * nkv * 8 <= 148)

    def rope_append(self, qkv, bias, rotary, nq, nkv, d, ctx, cache, q_norm=None, k_norm=None, norm_eps=0.0, dv=None,
                    own_kv=True, q_temp=None):
        """`qkv`: the stacked projections [T, (nq + 2 nkv) d] as a tensor or a PartialSum.
        With `q_norm` / `k_norm` (float32 [d]) every query / key head is RMS-normed with that weight before the
        rotation; `dv`: the values' head size if it is not `d` (cache rows hold the larger of the two);
        `own_kv` False: the rows hold queries only and nothing is stored; `q_temp` = (coef, every): the queries are
        multiplied by 1 + coef ln(floor((p + 1) / every) + 1) at position p.  A table whose cos and sin are made longer
        (`rotary.magnitude`) or cache rows longer than a head take the general kernel too."""
        if (q_norm is not None or k_norm is not None or (dv is not None and dv != d) or not own_kv or q_temp is not None
                or (rotary is not None and rotary.magnitude != 1.0) or (cache.kv is not None and cache.kv.shape[-1] != d)):
            return self._norm_rope_append(qkv, bias, rotary, nq, nkv, d, ctx, cache, q_norm, k_norm, norm_eps,
                                          d if dv is None else dv, own_kv, q_temp)
        partial, splits = None, 0
        if isinstance(qkv, PartialSum):
            partial, splits, dtype, device = qkv.parts, qkv.splits, qkv.dtype, qkv.parts.device
            T, width = qkv.shape
            qkv = None
        else:
            dtype, device = qkv.dtype, qkv.device
            T, width = qkv.shape
        _need(width == (nq + 2 * nkv) * d, "rope_append: qkv width does not fit the head counts")
        q_out = torch.empty((T, nq * d), dtype=dtype, device=device)
        write = bool(cache.writes and cache.kv is not None)
        kv, table = cache.kv, cache.block_table
        if write:
            _need(kv.dtype == dtype, f"rope_append: cache is {kv.dtype}, activations {dtype}")
        rot = 0 if rotary is None else int(rotary.rotary_dim)
        _need(rot <= d, "rope_append: rotary_dim exceeds the head size")
        _check(self.lib.ifx_rope_append(
            _ptr(qkv), _ptr(partial), splits, _ptr(bias), _ptr(None if rotary is None else rotary.inv_freq), rot,
            int(bool(rotary.interleaved)) if rotary is not None else 0,
            _ptr(ctx.positions), _ptr(ctx.token_req), _ptr(ctx.req_slot), _ptr(table),
            0 if table is None else table.shape[1], cache.page_size, 0 if kv is None else kv.shape[0],
            _ptr(kv), _ptr(q_out), T, nq, nkv, d, int(write), self.small_attention_grid(ctx, nkv), _DT[dtype],
            _stream()), "rope_append")
        self.launches += 1
        return q_out

    def _norm_rope_append(self, qkv, bias, rotary, nq, nkv, d, ctx, cache, q_norm, k_norm, norm_eps, dv, own_kv, q_temp=None):
        _need(bias is None, "rope_append: biases and head norms together are not built")
        partial, splits = None, 0
        if isinstance(qkv, PartialSum):
            partial, splits, dtype, device = qkv.parts, qkv.splits, qkv.dtype, qkv.parts.device
            T, width = qkv.shape
            qkv = None
        else:
            dtype, device = qkv.dtype, qkv.device
            T, width = qkv.shape
        src_kv = nkv if own_kv else 0
        _need(width == (nq + src_kv) * d + src_kv * dv, "rope_append: the rows' width does not fit the head counts")
        for w in (q_norm, k_norm):
            _need(w is None or (w.dtype == torch.float32 and w.numel() == d), "rope_append: a head norm weight is float32 [d]")
        q_out = torch.empty((T, nq * d), dtype=dtype, device=device)
        kv, table = cache.kv, cache.block_table
        write = bool(own_kv and cache.writes and kv is not None)
        d_row = d
        if write:
            _need(kv.dtype == dtype, f"rope_append: cache is {kv.dtype}, activations {dtype}")
            d_row = kv.shape[-1]
            _need(kv.shape[1] == 2 and kv.shape[2] == nkv and d_row >= max(d, dv), "rope_append: the cache does not fit the heads")
        rot = 0 if rotary is None else int(rotary.rotary_dim)
        _need(rot <= d, "rope_append: rotary_dim exceeds the head size")
        _check(self.lib.ifx_norm_rope_append_ex(
            _ptr(qkv), _ptr(partial), splits, _ptr(q_norm), _ptr(k_norm), ctypes.c_float(norm_eps),
            _ptr(None if rotary is None else rotary.inv_freq), rot,
            int(bool(rotary.interleaved)) if rotary is not None else 0, _ptr(ctx.positions), _ptr(ctx.token_req),
            _ptr(ctx.req_slot), _ptr(table), 0 if table is None else table.shape[1], cache.page_size,
            0 if kv is None else kv.shape[0], _ptr(kv if write else None), _ptr(q_out), T, nq, src_kv, nkv, d, dv, d_row,
            int(write), ctypes.c_float(1.0 if rotary is None else rotary.magnitude),
            ctypes.c_float(0.0 if q_temp is None else q_temp[0]), 0 if q_temp is None else int(q_temp[1]),
            _DT[dtype], _stream()), "rope_append (normed heads)")
        self.launches += 1
        return q_out

    def attention(self, q, nq, nkv, d, window, scale, ctx, cache, chunk=None, sink=False, dv=None):
        """Every token attends its request's keys up to its own position (or the last
        `window` of them) through the block table.  float32: the per-token kernel
        whose additions depend on the position only.  bfloat16: the tiled kernels,
        one launch for the prompt portions and one for the single decoded tokens.
        `chunk`: a query at position p sees keys from (p // chunk) * chunk on; `sink`: one more unit in the
        softmax's denominator (True), or exp of a learned number per head (a float32 tensor [nq]); `dv`: the values'
        head size if it is not `d`."""
        if (chunk or torch.is_tensor(sink) or sink or (dv is not None and dv != d)
                or (cache.kv is not None and cache.kv.shape[-1] != d)):      # cache rows longer than a head
            return self._attention_masked(q, nq, nkv, d, d if dv is None else dv, window, chunk, sink, scale, ctx, cache)
        T = q.shape[0]
        kv, table = cache.kv, cache.block_table
        _need(kv is not None and table is not None, "attention: the mixer has no key/value cache")
        _need(kv.dtype == q.dtype, f"attention: cache is {kv.dtype}, queries {q.dtype}")
        _need(d % 8 == 0 and d <= 256, f"attention: head size {d} is not a multiple of 8 up to 256")
        _need(q.is_contiguous() and q.shape[1] == nq * d, "attention: queries must be one [tokens, heads * size] block")
        out = torch.empty((T, nq * d), dtype=q.dtype, device=q.device)
        win = 0 if window is None else int(window)
        common = (cache.page_size, table.shape[1], kv.shape[0], win, ctypes.c_float(scale))
        tiled = q.dtype == torch.bfloat16 and bool(self.lib.ifx_attention_mma_supports(d))
        if "attn.prefill_tiles" not in ctx.extra:          # a step context built without the mixer as a provider
            for name, vals in self.attention_sections(ctx).items():
                ctx.extra[name] = torch.tensor(vals, dtype=torch.int32, device=q.device)
                ctx.extra_len[name] = len(vals)
        tiles, num_tiles = ctx.extra["attn.prefill_tiles"], ctx.extra_len["attn.prefill_tiles"] // 4
        decode_rows, decode_meta = ctx.extra["attn.decode_rows"], ctx.extra["attn.decode_meta"]
        if not tiled:
            self._attention_generic(q, kv, table, ctx, None, T, out, nq, nkv, d, common)
            return out
        if num_tiles and self.tensor_core_prefill and self.lib.ifx_attention_prefill_tcgen05_supports(
                d, cache.page_size):
            _check(self.lib.ifx_attention_prefill_tcgen05(
                _ptr(q), T, _ptr(kv), _ptr(table), _ptr(tiles), _ptr(ctx.req_slot), _ptr(out),
                num_tiles, nq, nkv, d, *common, _ptr(self.error_flag), _stream()),
                "attention (prompt portions, tcgen05)")
            self.launches += 1
        elif num_tiles:
            _check(self.lib.ifx_attention_prefill_bf16(
                _ptr(q), _ptr(kv), _ptr(table), _ptr(tiles), _ptr(ctx.req_slot), _ptr(out),
                num_tiles, nq, nkv, d, *common, int(ctx.max_kv_len), _ptr(self.error_flag), _stream()),
                "attention (prompt portions)")
            self.launches += 1
        n = ctx.extra_len["attn.decode_rows"]
        if n:
            if nq // nkv > 16:
                self._attention_generic(q, kv, table, ctx, decode_rows, n, out, nq, nkv, d, common)
                return out
            max_keys = int(ctx.max_kv_len if not win else min(win, ctx.max_kv_len))
            splits = self.decode_splits(n, nkv, max_keys, int(self.lib.ifx_attention_decode_max_splits(d, cache.page_size)))
            _check(self.lib.ifx_attention_decode_bf16(
                _ptr(q), _ptr(kv), _ptr(table), _ptr(decode_meta), _ptr(out), n, nq, nkv, d, *common, splits,
                max_keys, _ptr(self.error_flag), _stream()), "attention (decoded tokens)")
            self.launches += 1
        return out

    @staticmethod
    def decode_splits(num_tokens, nkv, max_keys, max_splits=8):
        """Into how many thread blocks (one cluster: 1, 2, 4, 8, or 16 where the kernel takes it) the
        key range of a decoded token is cut: as many blocks as the 148 SMs hold at once (two each), but
        at least 128 keys per block.  Clusters of 16 only while all of them fit on the SMs at once (measured:
        8.3 against 11.0 us for one token of the 7B shape at 4,096 keys, but 20 against 14 us for 16 clusters)."""
        want = max(1, 296 // max(1, num_tokens * nkv))           # all blocks resident at once: two a SM
        limit = max(1, min(want, max_keys // 128, max_splits))
        splits = 1
        while splits * 2 <= limit:
            splits *= 2
        if splits > 8 and num_tokens * nkv * splits > 148:
            splits = 8
        return splits

    def _attention_masked(self, q, nq, nkv, d, dv, window, chunk, sink, scale, ctx, cache):
        """Attention with a chunk mask, a sink or values of their own size: the per-token kernel."""
        T = q.shape[0]
        kv, table = cache.kv, cache.block_table
        _need(kv is not None and table is not None, "attention: the mixer has no key/value cache")
        _need(kv.dtype == q.dtype, f"attention: cache is {kv.dtype}, queries {q.dtype}")
        _need(q.is_contiguous() and q.shape[1] == nq * d, "attention: queries must be one [tokens, heads * size] block")
        d_row = kv.shape[-1]
        _need(kv.shape[1] == 2 and kv.shape[2] == nkv and d_row >= max(d, dv) and d_row % 8 == 0 and d_row <= 256,
              "attention: the cache does not fit the heads")
        out = torch.empty((T, nq * dv), dtype=q.dtype, device=q.device)
        win = 0 if window is None else int(window)
        sink_values = sink if torch.is_tensor(sink) else None
        if sink_values is not None:
            _need(sink_values.dtype == torch.float32 and sink_values.numel() == nq and sink_values.is_contiguous(),
                  "attention: the learned sink is float32 [heads]")
        if (q.dtype == torch.bfloat16 and d == dv == d_row and nq // nkv <= 16 and self.lib.ifx_attention_mma_supports(d)
                and os.environ.get("INFERFLUX_B200_MASKED_TILES", "1") != "0"):
            # the tiled kernels: prompt portions on mma.sync tiles, single tokens on the cluster kernel
            if "attn.prefill_tiles" not in ctx.extra:          # a step context built without the mixer as a provider
                for name, vals in self.attention_sections(ctx).items():
                    ctx.extra[name] = torch.tensor(vals, dtype=torch.int32, device=q.device)
                    ctx.extra_len[name] = len(vals)
            num_tiles = ctx.extra_len["attn.prefill_tiles"] // 4
            common = (cache.page_size, table.shape[1], kv.shape[0], win, int(chunk or 0),
                      int(sink_values is not None or bool(sink)), _ptr(sink_values), ctypes.c_float(scale))
            if num_tiles and self.tensor_core_prefill and self.lib.ifx_attention_prefill_tcgen05_supports(d, cache.page_size):
                _check(self.lib.ifx_attention_prefill_tcgen05_sink(
                    _ptr(q), T, _ptr(kv), _ptr(table), _ptr(ctx.extra["attn.prefill_tiles"]), _ptr(ctx.req_slot), _ptr(out),
                    num_tiles, nq, nkv, d, *common, _ptr(self.error_flag), _stream()),
                    "attention (masked, prompt portions, tcgen05)")
                self.launches += 1
            elif num_tiles:
                _check(self.lib.ifx_attention_prefill_bf16_sink(
                    _ptr(q), _ptr(kv), _ptr(table), _ptr(ctx.extra["attn.prefill_tiles"]), _ptr(ctx.req_slot), _ptr(out),
                    num_tiles, nq, nkv, d, *common, int(ctx.max_kv_len), _ptr(self.error_flag), _stream()),
                    "attention (masked, prompt portions)")
                self.launches += 1
            n = ctx.extra_len["attn.decode_rows"]
            if n:
                max_keys = int(ctx.max_kv_len)
                if win:
                    max_keys = min(max_keys, win)
                if chunk:
                    max_keys = min(max_keys, int(chunk))
                splits = self.decode_splits(n, nkv, max_keys, int(self.lib.ifx_attention_decode_max_splits(d, cache.page_size)))
                _check(self.lib.ifx_attention_decode_bf16_sink(
                    _ptr(q), _ptr(kv), _ptr(table), _ptr(ctx.extra["attn.decode_meta"]), _ptr(out), n, nq, nkv, d, *common,
                    splits, max_keys, _ptr(self.error_flag), _stream()), "attention (masked, decoded tokens)")
                self.launches += 1
            return out
        _check(self.lib.ifx_attention_generic_sink(
            _ptr(q), _ptr(kv), _ptr(table), _ptr(ctx.positions), _ptr(ctx.token_req), _ptr(ctx.req_slot), _ptr(None),
            _ptr(out), T, nq, nkv, d, dv, d_row, cache.page_size, table.shape[1], kv.shape[0],
            0 if window is None else int(window), int(chunk or 0), int(sink_values is not None or bool(sink)),
            _ptr(sink_values), ctypes.c_float(scale), _DT[q.dtype], _stream()), "attention (masked)")
        self.launches += 1
        return out

    def _attention_generic(self, q, kv, table, ctx, rows, count, out, nq, nkv, d, common):
        _check(self.lib.ifx_attention_generic(
            _ptr(q), _ptr(kv), _ptr(table), _ptr(ctx.positions), _ptr(ctx.token_req), _ptr(ctx.req_slot),
            _ptr(rows), _ptr(out), count, nq, nkv, d, *common, _DT[q.dtype], _stream()), "attention")
        self.launches += 1

    # ------------------------------------------- layers that norm a sublayer's output
    def postnorm_add(self, x, y, w_post, eps_post, w_next=None, eps_next=0.0, out_dtype=None, conv=None, cast_out=False,
                     groups=1, both=False):
        """x += y / rms(y) * w_post (x float32, in place).  With `w_next`, also returns the next norm of the
        updated rows, x / rms(x) * w_next in `out_dtype`: sum and both norms in one kernel.  With `cast_out`
        (and no `w_next`) it returns the updated rows themselves in `out_dtype`, for a sublayer that reads
        x without a norm.  `conv` =
        (weight [hidden, taps], taps, state, index, ctx), allowed when every request of the step brings one token
        (`ctx.max_span == 1`): the rows come back as h + conv(h) over time, and the state has moved on.
        `groups`: the next norm's root mean square is taken per group of the row.  `both` (with `conv`): returns
        (h, h + conv(h))."""
        if groups > 1 or both:
            return self._postnorm_add_groups(x, y, w_post, eps_post, w_next, eps_next, out_dtype, conv, groups, both)
        splits = 1
        if isinstance(y, PartialSum):                      # the slices are added in the same pass
            _need(tuple(y.shape) == tuple(x.shape), "postnorm_add: partial sums do not match x")
            out_dtype = out_dtype or y.dtype
            y, splits = y.parts, y.splits
        _need(x.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and tuple(y.shape[-2:]) == tuple(x.shape),
              "postnorm_add: x must be float32 and y of its shape")
        _need(w_post.dtype == torch.float32 and (w_next is None or w_next.dtype == torch.float32),
              "postnorm_add: norm weights must be float32")
        T, H = x.shape
        out = None if (w_next is None and not cast_out) else torch.empty((T, H), dtype=out_dtype or y.dtype, device=x.device)
        cw, taps, st_ptr, stride, treq, rslot = None, 0, ctypes.c_void_p(0), 0, None, None
        if conv is not None:
            cw, taps, state, index, ctx = conv
            _need(w_next is not None and ctx.max_span == 1 and tuple(cw.shape) == (H, taps) and cw.dtype == torch.float32,
                  "postnorm_add: the convolution is fused only into steps of single tokens")
            if taps > 1:
                _need(state is not None and state.dtype == torch.float32 and state.is_contiguous()
                      and tuple(state.shape[2:]) == (taps - 1, H) and 0 <= index < state.shape[1],
                      "postnorm_add: the state does not fit the convolution")
                stride = state.shape[1] * (taps - 1) * H
                st_ptr = ctypes.c_void_p(state.data_ptr() + 4 * index * (taps - 1) * H)
            treq, rslot = ctx.token_req, ctx.req_slot
        _check(self.lib.ifx_postnorm_add_rmsnorm(
            _ptr(x), _ptr(y), _ptr(w_post), ctypes.c_float(eps_post), _ptr(w_next), ctypes.c_float(eps_next), _ptr(out),
            T, H, _DT[y.dtype], _DT[(out_dtype or y.dtype)], splits, _ptr(cw), taps, st_ptr, ctypes.c_longlong(stride),
            _ptr(treq), _ptr(rslot), _stream()), "postnorm_add")
        self.launches += 1
        return out

    def _postnorm_add_groups(self, x, y, w_post, eps_post, w_next, eps_next, out_dtype, conv, groups, both):
        splits = 1
        if isinstance(y, PartialSum):
            _need(tuple(y.shape) == tuple(x.shape), "postnorm_add: partial sums do not match x")
            out_dtype = out_dtype or y.dtype
            y, splits = y.parts, y.splits
        _need(x.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and tuple(y.shape[-2:]) == tuple(x.shape),
              "postnorm_add: x must be float32 and y of its shape")
        _need(w_next is not None and w_post.dtype == torch.float32 and w_next.dtype == torch.float32,
              "postnorm_add: a norm over groups needs both float32 norm weights")
        T, H = x.shape
        out_dtype = out_dtype or y.dtype
        out = torch.empty((T, H), dtype=out_dtype, device=x.device)
        out2, cw, taps, st_ptr, stride, treq, rslot = None, None, 0, ctypes.c_void_p(0), 0, None, None
        if conv is not None:
            cw, taps, state, index, ctx = conv
            _need(ctx.max_span == 1 and tuple(cw.shape) == (H, taps) and cw.dtype == torch.float32,
                  "postnorm_add: the convolution is fused only into steps of single tokens")
            if taps > 1:
                _need(state is not None and state.dtype == torch.float32 and tuple(state.shape[2:]) == (taps - 1, H)
                      and state.stride(3) == 1 and state.stride(2) == H and 0 <= index < state.shape[1],
                      "postnorm_add: the state does not fit the convolution")
                stride = state.stride(0)
                st_ptr = ctypes.c_void_p(state.data_ptr() + 4 * index * state.stride(1))
            treq, rslot = ctx.token_req, ctx.req_slot
            out2 = torch.empty((T, H), dtype=out_dtype, device=x.device)
        _check(self.lib.ifx_groupnorm_stream(
            _ptr(x), _ptr(y), _ptr(w_post), ctypes.c_float(eps_post), _ptr(w_next), ctypes.c_float(eps_next), int(groups),
            _ptr(out), _ptr(out2), T, H, _DT[y.dtype], _DT[out_dtype], splits, _ptr(cw), taps, st_ptr,
            ctypes.c_longlong(stride), _ptr(treq), _ptr(rslot), _stream()), "postnorm_add (groups)")
        self.launches += 1
        if conv is None:
            return out
        return (out, out2) if both else out2

    def residual_add_scaled(self, x, a, b, scale, out_dtype=None):
        """x += scale * (a + b) (x float32, in place; b may be None; a and b tensors of x's shape or PartialSums).  With
        `out_dtype` also returns the updated rows in that dtype."""
        T, H = x.shape
        _need(x.dtype == torch.float32 and x.is_contiguous(), "residual_add_scaled: x must be contiguous float32")

        def operand(v):
            if v is None:
                return None, 0, 1
            if isinstance(v, PartialSum):
                _need(tuple(v.shape) == (T, H), "residual_add_scaled: partial sums do not match x")
                return v.parts, 0, v.splits
            _need(tuple(v.shape) == (T, H) and v.is_contiguous(), "residual_add_scaled: an operand does not match x")
            return v, _DT[v.dtype], 1
        pa, da, sa = operand(a)
        pb, db, sb = operand(b)
        out = None if out_dtype is None else torch.empty((T, H), dtype=out_dtype, device=x.device)
        _check(self.lib.ifx_residual_add_scaled(_ptr(x), _ptr(pa), da, sa, _ptr(pb), db, sb, ctypes.c_float(scale), _ptr(out),
                                                0 if out is None else _DT[out_dtype], T, H, _stream()), "residual_add_scaled")
        self.launches += 1
        return out

    def scale_(self, values, factor):
        """values *= factor, in place (float32)."""
        _need(values.dtype == torch.float32 and values.is_contiguous(), "scale_: contiguous float32 values")
        _check(self.lib.ifx_scale_f32(_ptr(values), ctypes.c_longlong(values.numel()), ctypes.c_float(factor), _stream()), "scale_")
        self.launches += 1

    def gelu_mul_table(self, z, table, token_ids, first_column):
        """gelu_tanh(z) * table[token, first_column : first_column + z.shape[1]], in z's dtype."""
        T, dim = z.shape
        _need(z.is_contiguous() and table.is_contiguous() and table.dtype == z.dtype and token_ids.numel() == T
              and first_column + dim <= table.shape[1], "gelu_mul_table: rows and table of one dtype, columns inside the table")
        out = torch.empty_like(z)
        _check(self.lib.ifx_gelu_mul_table(_ptr(z), _ptr(table), _ptr(token_ids), table.shape[1], int(first_column),
                                           table.shape[0], _ptr(out), T, dim, _DT[z.dtype], _stream()), "gelu_mul_table")
        self.launches += 1
        return out

    def rmsnorm_columns(self, rows, col0, n, w, eps):
        """Columns col0 .. col0 + n of `rows`, RMS-normed with weight `w` (float32), as a tensor of their own."""
        T, ld = rows.shape
        _need(rows.is_contiguous() and w.dtype == torch.float32 and w.numel() == n and col0 + n <= ld,
              "rmsnorm_columns: the columns must lie inside contiguous rows")
        out = torch.empty((T, n), dtype=rows.dtype, device=rows.device)
        _check(self.lib.ifx_latent_norm_append(
            _ptr(rows), ld, int(col0), _ptr(w), ctypes.c_float(eps), _ptr(None), _ptr(None), _ptr(None), _ptr(None), 0, 0, 0,
            _ptr(None), _ptr(out), T, n, _DT[rows.dtype], _stream()), "rmsnorm_columns")
        self.launches += 1
        return out

    def concat_cast(self, a, b, dtype):
        """[a; b] along the columns, from two float32 tensors into `dtype`."""
        _need(a.dtype == torch.float32 and b.dtype == torch.float32 and a.shape == b.shape and a.is_contiguous()
              and b.is_contiguous(), "concat_cast: two float32 tensors of one shape")
        T, H = a.shape
        out = torch.empty((T, 2 * H), dtype=dtype, device=a.device)
        _check(self.lib.ifx_concat_cast(_ptr(a), _ptr(b), _ptr(out), T, H, _DT[dtype], _stream()), "concat_cast")
        self.launches += 1
        return out

    def xielu(self, z, a_pos, a_neg):
        """a_pos z^2 + z/2 above zero, a_neg (e^z - 1 - z) + z/2 below, element by element, in float32."""
        splits, out_dtype = 1, z.dtype
        if isinstance(z, PartialSum):                      # a K-split product: the slices are added first, in the same pass
            out_dtype, splits, z = z.dtype, z.splits, z.parts
        _need(z.is_contiguous(), "xielu: contiguous input")
        out = torch.empty(tuple(z.shape[-2:]), dtype=out_dtype, device=z.device)
        _check(self.lib.ifx_xielu(_ptr(z), _ptr(out), ctypes.c_longlong(out.numel()), ctypes.c_float(a_pos),
                                  ctypes.c_float(a_neg), _DT[z.dtype], _DT[out_dtype], splits, _stream()), "xielu")
        self.launches += 1
        return out

    def softcap(self, logits, cap):
        """logits <- cap tanh(logits / cap), in place (float32)."""
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "softcap: float32 logits")
        _check(self.lib.ifx_softcap(_ptr(logits), ctypes.c_longlong(logits.numel()), ctypes.c_float(cap), _stream()),
               "softcap")
        self.launches += 1

    def short_conv(self, h, w, taps, state, index, ctx, add_input=True, bias=None, act=None, columns=None):
        """h + causal depthwise convolution of h over each request's tokens; `state[:, index]` (float32
        [slots, convolutions, taps - 1, channels]) brings the inputs before the step and takes the last ones.
        `add_input` False: the convolution alone; `bias` (float32 [channels]) is added and `act` ("silu") applied
        behind it; `columns` = (first, count): the convolution runs over those columns of `h` and returns them alone."""
        T, width = h.shape
        col0, C = (0, width) if columns is None else (int(columns[0]), int(columns[1]))
        _need(h.is_contiguous() and w.dtype == torch.float32 and tuple(w.shape) == (C, taps) and w.is_contiguous()
              and 0 <= col0 and col0 + C <= width and act in (None, "silu")
              and (bias is None or (bias.dtype == torch.float32 and bias.numel() == C)), "short_conv: bad operands")
        st_ptr, stride = ctypes.c_void_p(0), 0
        if taps > 1:
            _need(state is not None and state.dtype == torch.float32 and tuple(state.shape[2:]) == (taps - 1, C)
                  and state.stride(3) == 1 and state.stride(2) == C and 0 <= index < state.shape[1],
                  "short_conv: the state does not fit the convolution")
            stride = state.stride(0)                       # a slot's rows may be part of a longer state row
            st_ptr = ctypes.c_void_p(state.data_ptr() + 4 * index * state.stride(1))
        out = torch.empty((T, C), dtype=h.dtype, device=h.device)
        _check(self.lib.ifx_short_conv_ex(ctypes.c_void_p(h.data_ptr() + col0 * h.element_size()), ctypes.c_longlong(width),
                                          _ptr(w), _ptr(bias), st_ptr, ctypes.c_longlong(stride), _ptr(ctx.token_req),
                                          _ptr(ctx.req_slot), _ptr(ctx.cu_seqlens), _ptr(out), T, ctx.num_requests, C,
                                          taps, int(ctx.max_span > 1), ctypes.c_float(1.0 if add_input else 0.0),
                                          int(act == "silu"), _DT[h.dtype], _stream()), "short_conv")
        self.launches += 1 + int(taps > 1 and ctx.max_span > 1)
        return out

    # -------------------------------------------------------- latent attention
    LATENT_TILE = 64           # tokens per work item of the tiled latent attention kernel

    def latent_attention_sections(self, ctx):
        """latent.items[P, 4] = (slot, first flat token, tokens, first position): every span in pieces of up
        to 64 tokens; a decoded token is an item of one."""
        items, base = [], 0
        for (start, n), slot in zip(ctx.spans, ctx.slots_host):
            for off in range(0, n, self.LATENT_TILE):
                items.extend((int(slot), base + off, min(self.LATENT_TILE, n - off), start + off))
            base += n
        return {"latent.items": items}

    def linear_heads(self, a, w, heads, k, n, w_is_nk, a_head_stride=None, out=None, out_head_stride=None):
        """One small product per head, heads side by side in the rows of `a` [T, >= heads * k]:
        out[:, h n:(h + 1) n] = a[:, h k:(h + 1) k] . W_h^T with W_h = w[h n:(h + 1) n] of [n, k] (w_is_nk), or
        a[:, h k:(h + 1) k] . W_h with W_h = w[h k:(h + 1) k] of [k, n].  bfloat16, through the library.
        `a_head_stride`: a head's columns begin that far apart in `a` (default k); `out` with `out_head_stride`:
        the heads' results go into columns of that tensor, that far apart."""
        T, lda = a.shape
        sa = k if a_head_stride is None else int(a_head_stride)
        _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous(),
              "linear_heads: contiguous bfloat16 operands")
        _need(tuple(w.shape) == ((heads * n, k) if w_is_nk else (heads * k, n)) and sa >= k and lda >= (heads - 1) * sa + k,
              "linear_heads: shapes do not fit")
        so = n if out_head_stride is None else int(out_head_stride)
        if out is None:
            out = torch.empty((T, heads * so), dtype=torch.bfloat16, device=a.device)
        _need(out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[0] == T and so >= n
              and out.shape[1] >= (heads - 1) * so + n, "linear_heads: the output does not fit")
        ldw = k if w_is_nk else n
        _check(self.lib.ifx_gemm_cublas_bf16_batched(
            _ptr(a), _LL(lda), _LL(sa), _ptr(w), _LL(ldw), _LL(k * n), _ptr(out), _LL(out.shape[1]), _LL(so), T, n, k, heads,
            int(bool(w_is_nk)), _stream()), "linear_heads")
        self.library_calls += 1
        return out

    def latent_norm_append(self, rows, col0, rank, w, eps, ctx, cache):
        """The latent of every token: columns col0 .. col0 + rank of `rows`, RMS-normed with weight `w`,
        written to the cache at the token's position."""
        T, ld = rows.shape
        kv, table = cache.kv, cache.block_table
        _need(kv is not None and table is not None and kv.dtype == rows.dtype, "latent_norm_append: no cache of the run's dtype")
        _need(kv.shape[1] == 1 and kv.shape[2] == 1 and kv.shape[4] == rank, "latent_norm_append: the cache is not one latent plane")
        write = bool(cache.writes)
        _check(self.lib.ifx_latent_norm_append(
            _ptr(rows), ld, col0, _ptr(w), ctypes.c_float(eps), _ptr(ctx.positions), _ptr(ctx.token_req),
            _ptr(ctx.req_slot), _ptr(table), table.shape[1], cache.page_size, kv.shape[0], _ptr(kv if write else None),
            _ptr(None), T, rank, _DT[rows.dtype], _stream()), "latent_norm_append")
        self.launches += 1

    def latent_rope_append(self, rows, col0, rank, rot, w, eps, q, heads, dim, rotary, ctx, cache, vdim=None):
        """The cached row of every token: [columns col0 .. + rank of `rows`, RMS-normed with `w`; the `rot` columns
        behind them, turned by the token's position], written at the token's position.  Returns `q`
        [T, heads (dim + rot)] with every head's last `rot` elements turned the same way (in place), or, where the
        tiled attention kernel takes the sizes (`vdim` given), a `TurnedQueries`: the turned parts then lie in the
        rows of queries in latent space, [T, heads (rank + rot)], whose other columns `latent_attention` fills."""
        T, ld = rows.shape
        kv, table = cache.kv, cache.block_table
        _need(kv is not None and table is not None and kv.dtype == rows.dtype and q.dtype == rows.dtype,
              "latent_rope_append: no cache of the run's dtype")
        _need(kv.shape[1] == 1 and kv.shape[2] == 1 and kv.shape[4] == rank + rot,
              "latent_rope_append: the cache is not one plane of latent and turned part")
        _need(rows.is_contiguous() and q.is_contiguous() and q.shape[0] == T and q.shape[1] >= heads * (dim + rot),
              "latent_rope_append: contiguous rows")
        used, inter, mag, freq = 0, 0, 1.0, None
        if rot and rotary is not None:
            used, inter, mag, freq = int(rotary.rotary_dim), int(bool(rotary.interleaved)), float(rotary.magnitude), rotary.inv_freq
            _need(used <= rot and freq.dtype == torch.float32 and freq.numel() == used // 2,
                  "latent_rope_append: the table does not fit the turned part")
        write = bool(cache.writes)
        dst, ld_dst, head_stride, offset, result = q, q.shape[1], dim + rot, dim, q
        if (rot and vdim is not None and self.latent_tiles and rows.dtype == torch.bfloat16 and dim % 8 == 0 and vdim % 8 == 0
                and q.shape[1] % 8 == 0 and self.lib.ifx_latent_attention_mma_supports_rot(rank, rot)):
            dst = torch.empty((T, heads * (rank + rot)), dtype=torch.bfloat16, device=rows.device)
            ld_dst, head_stride, offset, result = heads * (rank + rot), rank + rot, rank, TurnedQueries(q, dst)
        _check(self.lib.ifx_latent_rope_append(
            _ptr(rows), ld, int(col0), _ptr(w), ctypes.c_float(eps), _ptr(q), q.shape[1], _ptr(dst), ld_dst, head_stride, offset,
            _ptr(freq), used, inter, ctypes.c_float(mag), _ptr(ctx.positions), _ptr(ctx.token_req), _ptr(ctx.req_slot),
            _ptr(table), table.shape[1], cache.page_size, kv.shape[0], _ptr(kv if write else None), T, rank, rot, heads, dim,
            _DT[rows.dtype], _stream()), "latent_rope_append")
        self.launches += 1
        return result

    def latent_attention(self, q_rows, w_uk, w_uv, sinks, heads, dim, vdim, rank, window, scale, ctx, cache, rot=0):
        """Attention over cached latents (see csrc/latent_attention.cu).  `q_rows`: [T, >= heads * (dim + rot)], the
        queries in its first columns, every head's `rot` turned elements behind its `dim` plain ones; cached rows
        are [latent of `rank`; turned key part of `rot`].  Returns [T, heads * vdim]."""
        turned = None
        if isinstance(q_rows, TurnedQueries):
            q_rows, turned = q_rows.rows, q_rows.latent
        T, ldq = q_rows.shape
        kv, table = cache.kv, cache.block_table
        _need(kv is not None and table is not None and kv.dtype == q_rows.dtype, "latent_attention: no cache of the run's dtype")
        _need(q_rows.is_contiguous() and w_uk.is_contiguous() and w_uv.is_contiguous(), "latent_attention: contiguous operands")
        _need(tuple(w_uk.shape) == (heads * dim, rank) and tuple(w_uv.shape) == (heads * vdim, rank),
              "latent_attention: the up-projections do not fit the sizes")
        _need(kv.shape[4] == rank + rot and ldq >= heads * (dim + rot), "latent_attention: rows do not hold the turned part")
        if turned is not None:
            return self._latent_attention_tiles(q_rows, w_uk, w_uv, sinks, heads, dim, vdim, rank, window, scale, ctx, cache,
                                                rot=rot, ql=turned)
        if rot:
            out = torch.empty((T, heads * vdim), dtype=q_rows.dtype, device=q_rows.device)
            _check(self.lib.ifx_latent_attention_generic_rot(
                _ptr(q_rows), ldq, _ptr(w_uk), _ptr(w_uv), _ptr(sinks), _ptr(kv), _ptr(table), _ptr(ctx.positions),
                _ptr(ctx.token_req), _ptr(ctx.req_slot), _ptr(None), _ptr(out), T, heads, dim, vdim, rank, cache.page_size,
                table.shape[1], kv.shape[0], 0 if window is None else int(window), ctypes.c_float(scale), int(rot),
                _DT[q_rows.dtype], _stream()), "latent_attention (turned part)")
            self.launches += 1
            return out
        if (self.latent_tiles and q_rows.dtype == torch.bfloat16 and self.lib.ifx_latent_attention_mma_supports(rank)
                and dim % 8 == 0 and vdim % 8 == 0 and ldq % 8 == 0):
            return self._latent_attention_tiles(q_rows, w_uk, w_uv, sinks, heads, dim, vdim, rank, window, scale, ctx, cache)
        out = torch.empty((T, heads * vdim), dtype=q_rows.dtype, device=q_rows.device)
        _check(self.lib.ifx_latent_attention_generic(
            _ptr(q_rows), ldq, _ptr(w_uk), _ptr(w_uv), _ptr(sinks), _ptr(kv), _ptr(table), _ptr(ctx.positions),
            _ptr(ctx.token_req), _ptr(ctx.req_slot), _ptr(None), _ptr(out), T, heads, dim, vdim, rank, cache.page_size,
            table.shape[1], kv.shape[0], 0 if window is None else int(window), ctypes.c_float(scale), _DT[q_rows.dtype],
            _stream()), "latent_attention")
        self.launches += 1
        return out

    def _latent_attention_tiles(self, q_rows, w_uk, w_uv, sinks, heads, dim, vdim, rank, window, scale, ctx, cache, rot=0,
                                ql=None):
        """bfloat16: queries into latent space (a product per head), the tensor-core kernel over cached latents
        with all heads of a token tile in one block, the value projection per head on the weighted latents.
        With `rot`, `ql` [T, heads (rank + rot)] holds the turned query parts already, behind the columns that the
        product per head fills."""
        T = q_rows.shape[0]
        kv, table = cache.kv, cache.block_table
        if "latent.items" not in ctx.extra:                # a step context built without the mixer as a provider
            vals = self.latent_attention_sections(ctx)["latent.items"]
            ctx.extra["latent.items"] = torch.tensor(vals, dtype=torch.int32, device=q_rows.device)
            ctx.extra_len["latent.items"] = len(vals)
        items, num_items = ctx.extra["latent.items"], ctx.extra_len["latent.items"] // 4
        if rot:
            self.linear_heads(q_rows, w_uk, heads, dim, rank, w_is_nk=False, a_head_stride=dim + rot, out=ql,
                              out_head_stride=rank + rot)
        else:
            ql = self.linear_heads(q_rows, w_uk, heads, dim, rank, w_is_nk=False)           # [T, heads * rank]
        win = 0 if window is None else int(window)
        splits = 1
        max_keys = int(ctx.max_kv_len if not win else min(win, ctx.max_kv_len))
        if ctx.max_span == 1:                              # decoded tokens only: cut the keys so that the SMs fill
            blocks = num_items * -(-heads // 64)                 # about four warps a SM, at least two key tiles each
            splits = max(1, min(592 // max(1, blocks), max_keys // 64, 64))
        else:
            # prompt portions: a block walks its keys tile after tile, and the last tokens' blocks walk all of them;
            # while the grid does not fill the SMs twice over (three blocks a SM), cut every block's keys in 2..4
            hc = min(heads, 64)
            qt = max(1, min(64 // hc, self.LATENT_TILE, ctx.max_span))
            blocks = -(-T // qt) * -(-heads // 64)
            splits = max(1, min(888 // max(1, blocks), max_keys // 256, 4))
        ws = None
        if splits > 1:
            ws = torch.empty(int(self.lib.ifx_latent_attention_mma_workspace(T * heads, rank, splits)), dtype=torch.uint8,
                             device=q_rows.device)
        olat = torch.empty((T, heads * rank), dtype=torch.bfloat16, device=q_rows.device)
        _check(self.lib.ifx_latent_attention_mma_rot(
            _ptr(ql), _ptr(kv), _ptr(table), _ptr(items), num_items, int(min(self.LATENT_TILE, ctx.max_span)), _ptr(sinks),
            _ptr(olat), _ptr(ws), T, heads, rank, int(rot), cache.page_size, table.shape[1], kv.shape[0], win,
            ctypes.c_float(scale), splits, _stream()), "latent_attention (tiles)")
        self.launches += 1 + int(splits > 1)
        return self.linear_heads(olat, w_uv, heads, rank, vdim, w_is_nk=True)               # [T, heads * vdim]

    # ------------------------------------------------- recurrence with matrix state
    def cast_rows(self, x, dtype):
        """float32 rows in the run's dtype (the rows themselves when that is float32)."""
        if dtype == torch.float32:
            return x
        _need(x.dtype == torch.float32 and x.is_contiguous(), "cast_rows: contiguous float32 rows")
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
        _check(self.lib.ifx_cast_rows(_ptr(x), _ptr(out), ctypes.c_longlong(x.numel()), _DT[dtype], _stream()), "cast_rows")
        self.launches += 1
        return out

    def tanh(self, z):
        """tanh of every element, in place."""
        _need(z.is_contiguous(), "tanh: contiguous input")
        _check(self.lib.ifx_tanh_rows(_ptr(z), ctypes.c_longlong(z.numel()), _DT[z.dtype], _stream()), "tanh")
        self.launches += 1
        return z

    def token_shift_mix(self, x, mu, state, prev_offset, ctx, out_dtype):
        """mixes[m, t] = x[t] + (x[t - 1] - x[t]) * mu[m] for the float32 rows `x` [T, C] and `mu` [M, C]; the row
        before a span's first one is `state[slot, prev_offset : prev_offset + C]` (float32; zeros at a sequence's
        start).  The state is not changed here: `wkv_scan` leaves the step's last row there."""
        T, C = x.shape
        _need(x.dtype == torch.float32 and x.is_contiguous() and mu.dtype == torch.float32 and mu.is_contiguous()
              and mu.shape[1] == C, "token_shift_mix: float32 rows and weights of one width")
        _need(state is not None and state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2
              and prev_offset + C <= state.shape[1], "token_shift_mix: the state does not hold a row")
        out = torch.empty((mu.shape[0], T, C), dtype=out_dtype, device=x.device)
        _check(self.lib.ifx_token_shift_mix(
            _ptr(x), _ptr(mu), ctypes.c_void_p(state.data_ptr() + 4 * prev_offset), ctypes.c_longlong(state.shape[1]),
            _ptr(ctx.token_req), _ptr(ctx.req_slot), _ptr(ctx.cu_seqlens), _ptr(out), T, C, mu.shape[0], _DT[out_dtype],
            _stream()), "token_shift_mix")
        self.launches += 1
        return out

    def wkv_scan(self, r, k, v, w_raw, g, w0, u, norm_w, eps, heads, dim, state, prev_offset, x, ctx, out_dtype):
        """The recurrence of csrc/wkv.cu over every request's tokens.  r, k, v, w_raw, g: float32 [T, heads * dim], each
        contiguous or a column block of a wider matrix (all with the same distance between rows);
        `state`: float32 [slots, heads * dim * dim + C], the matrices first, then the last input row, both moved on.
        Returns out / rms(out) per head * norm_w * silu(g) in `out_dtype`."""
        T, HD = r.shape
        C = x.shape[1]
        ld, ld_w = max(int(r.stride(0)), HD), max(int(w_raw.stride(0)), HD)
        for t in (r, k, v, w_raw, g):
            _need(t.dtype == torch.float32 and tuple(t.shape) == (T, HD) and t.stride(1) == 1
                  and (T == 1 or t.stride(0) == (ld_w if t is w_raw else ld)),
                  "wkv_scan: float32 [T, heads * dim] inputs; r, k, v and g with one distance between rows")
        for t in (w0, u, norm_w):
            _need(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == HD, "wkv_scan: float32 constants of heads * dim")
        _need(HD == heads * dim and prev_offset == heads * dim * dim and state.dtype == torch.float32 and state.is_contiguous()
              and state.dim() == 2 and state.shape[1] == prev_offset + C and x.dtype == torch.float32 and x.is_contiguous(),
              "wkv_scan: the state does not fit the sizes")
        scratch = torch.empty((T, HD), dtype=torch.float32, device=r.device)
        y = torch.empty((T, HD), dtype=out_dtype, device=r.device)
        _check(self.lib.ifx_wkv_scan(
            _ptr(r), _ptr(k), _ptr(v), _ptr(w_raw), _ptr(g), _ptr(w0), _ptr(u), _ptr(norm_w), ctypes.c_float(eps),
            _ptr(state), ctypes.c_void_p(state.data_ptr() + 4 * prev_offset), ctypes.c_longlong(state.shape[1]), _ptr(x), C,
            _ptr(ctx.cu_seqlens), _ptr(ctx.req_slot), _ptr(scratch), _ptr(y), ctx.num_requests, T, heads, dim, ld, ld_w, _DT[out_dtype],
            _stream()), "wkv_scan")
        self.launches += 1
        return y

    def delta_rule_scan(self, proj, w_raw, w0, a_bias, norm_w, eps, heads, dim, state, ctx, out_dtype):
        """The recurrence of csrc/delta_rule.cu over every request's tokens.  `proj`: float32 [T, 5 heads dim], the
        projections r, k, v, g, a side by side; `w_raw`: float32 [T, heads dim]; `state`: float32 [slots, >= heads dim
        dim] (rows may be further apart), the matrices [head, key channel, value channel], moved on.  Returns
        out / rms(out) per head * norm_w * sigmoid(g) in `out_dtype`."""
        T, HD = proj.shape[0], heads * dim
        _need(proj.dtype == torch.float32 and proj.is_contiguous() and proj.shape[1] >= 5 * HD and w_raw.dtype == torch.float32
              and w_raw.is_contiguous() and tuple(w_raw.shape) == (T, HD), "delta_rule_scan: float32 projections")
        for t in (w0, a_bias, norm_w):
            _need(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == HD, "delta_rule_scan: float32 constants of heads * dim")
        _need(state is not None and state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1
              and state.shape[1] >= HD * dim, "delta_rule_scan: the state does not fit the sizes")
        scratch = torch.empty(int(self.lib.ifx_delta_rule_scratch_floats(T, heads, dim)), dtype=torch.float32, device=proj.device)
        y = torch.empty((T, HD), dtype=out_dtype, device=proj.device)
        _check(self.lib.ifx_delta_rule_scan(
            _ptr(proj), proj.shape[1], _ptr(w_raw), _ptr(w0), _ptr(a_bias), _ptr(norm_w), ctypes.c_float(eps), _ptr(state),
            ctypes.c_longlong(state.stride(0)), _ptr(ctx.cu_seqlens), _ptr(ctx.req_slot), _ptr(scratch), _ptr(y),
            ctx.num_requests, T, heads, dim, _DT[out_dtype], _stream()), "delta_rule_scan")
        self.launches += 3
        return y

    # ------------------------------------------------------- mixture of experts
    def moe_route(self, z, correction, top, of_chosen=False, kind=None, floor=0.0):
        """(ids int32 [T, top], weights float32 [T, top]) from router logits z float32 [T, n]: softmax scores; the
        `top` largest of score + correction are chosen, their weights are the scores.  `of_chosen`: the `top`
        largest of z + correction are chosen, and the weights are the softmax over the chosen logits alone.
        `kind` = "sigmoid_normalized": scores = sigmoid(z), the `top` largest of score + correction are chosen, and the
        weights are the chosen scores divided by (their sum + floor)."""
        _need(kind in (None, "sigmoid_normalized"), f"moe_route: unknown kind {kind!r}")
        T, n = z.shape
        _need(z.dtype == torch.float32 and z.is_contiguous() and (correction is None or (correction.dtype == torch.float32
              and correction.numel() == n)), "moe_route: float32 logits and corrections")
        ids = torch.empty((T, top), dtype=torch.int32, device=z.device)
        weights = torch.empty((T, top), dtype=torch.float32, device=z.device)
        _check(self.lib.ifx_moe_route_kind(_ptr(z), _ptr(correction), _ptr(ids), _ptr(weights), T, n, int(top),
                                           2 if kind == "sigmoid_normalized" else int(bool(of_chosen)), ctypes.c_float(floor),
                                           _stream()), "moe_route")
        self.launches += 1
        return ids, weights

    def moe_experts(self, h, w_up, w_down, ids, weights, experts, out_dtype, glu=None):
        """sum over a token's choices of weight * W_down[e] relu(W_up[e] h)^2, or weight * h for e >= experts.
        w_up [experts, ff, width], w_down [experts, width, ff] in h's dtype.  `glu` = (limit, slope): w_up is
        [experts, 2 ff, width], an expert's gate rows above its up rows, and the activation is
        g sigmoid(slope g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit); a third number replaces
        the 1 (limit inf, slope 1 and 0 give silu(gate) * up)."""
        T, width = h.shape
        top = ids.shape[1]
        if glu is not None and len(glu) == 2:
            glu = (glu[0], glu[1], 1.0)
        if glu is not None:
            _need(experts > 0 and w_up.shape[1] % 2 == 0, "moe_experts: gated experts need gate and up rows")
            ff = w_up.shape[1] // 2
            _need(h.is_contiguous() and w_up.dtype == h.dtype and w_down.dtype == h.dtype and w_up.is_contiguous()
                  and w_down.is_contiguous() and tuple(w_up.shape) == (experts, 2 * ff, width)
                  and tuple(w_down.shape) == (experts, width, ff), "moe_experts: stacked expert weights in the activations' dtype")
            if (h.dtype == torch.bfloat16 and T * top >= self.MOE_TILES_MIN_PAIRS and width % 8 == 0 and ff % 8 == 0
                    and h.data_ptr() % 16 == 0 and os.environ.get("INFERFLUX_B200_MOE_TILES", "1") != "0"):
                return self._moe_experts_tiles(h, w_up, w_down, ids, weights, experts, out_dtype, glu=glu)
            act = torch.empty((T * top, ff), dtype=h.dtype, device=h.device)
            out = torch.empty((T, width), dtype=out_dtype, device=h.device)
            _check(self.lib.ifx_moe_experts_glu(_ptr(h), _ptr(w_up), _ptr(w_down), _ptr(ids), _ptr(weights), _ptr(act), _ptr(out),
                                                T, top, int(experts), width, ff, _DT[h.dtype], _DT[out_dtype], 1,
                                                ctypes.c_float(glu[0]), ctypes.c_float(glu[1]), ctypes.c_float(glu[2]),
                                                _stream()), "moe_experts (gated)")
            self.launches += 2
            return out
        ff = w_up.shape[1] if experts else 1
        _need(h.is_contiguous() and (not experts or (w_up.dtype == h.dtype and w_down.dtype == h.dtype and w_up.is_contiguous()
              and w_down.is_contiguous() and tuple(w_up.shape) == (experts, ff, width) and tuple(w_down.shape) == (experts, width, ff))),
              "moe_experts: stacked expert weights in the activations' dtype")
        if (experts and h.dtype == torch.bfloat16 and T * top >= self.MOE_TILES_MIN_PAIRS and width % 8 == 0 and ff % 8 == 0
                and h.data_ptr() % 16 == 0 and os.environ.get("INFERFLUX_B200_MOE_TILES", "1") != "0"):
            return self._moe_experts_tiles(h, w_up, w_down, ids, weights, experts, out_dtype)
        act = torch.empty((T * top, ff), dtype=h.dtype, device=h.device)
        out = torch.empty((T, width), dtype=out_dtype, device=h.device)
        _check(self.lib.ifx_moe_experts(_ptr(h), _ptr(w_up if experts else None), _ptr(w_down if experts else None), _ptr(ids),
                                        _ptr(weights), _ptr(act), _ptr(out), T, top, int(experts), width, ff, _DT[h.dtype],
                                        _DT[out_dtype], _stream()), "moe_experts")
        self.launches += 2 if experts else 1
        return out

    # From this many (token, choice) pairs on, the experts run as sorted 128-row tiles on the tensor cores.
    MOE_TILES_MIN_PAIRS = 512

    def _moe_experts_tiles(self, h, w_up, w_down, ids, weights, experts, out_dtype, glu=None):
        """bfloat16, many tokens: pairs sorted by expert into stretches of whole 128-row tiles, two grouped tcgen05
        products (the activation, relu^2 or the gated one of `glu` over tiles of 128 gate rows and their 128 up rows, in
        the first one's epilogue, the pair's weight in the second's), then the sum per token."""
        T, width = h.shape
        top, ff = ids.shape[1], w_up.shape[1] // (2 if glu is not None else 1)
        pairs = T * top
        cap = int(self.lib.ifx_moe_sorted_rows(pairs, int(experts)))
        dev = h.device
        row_pair = torch.empty(cap, dtype=torch.int32, device=dev)
        row_scale = torch.empty(cap, dtype=torch.float32, device=dev)
        tile_group = torch.empty(cap // 128, dtype=torch.int32, device=dev)
        pair_row = torch.empty(pairs, dtype=torch.int32, device=dev)
        _check(self.lib.ifx_moe_sort(_ptr(ids), _ptr(weights), pairs, int(experts), _ptr(row_pair), _ptr(row_scale),
                                     _ptr(tile_group), _ptr(pair_row), cap, _stream()), "moe_sort")
        rows = torch.empty((cap, width), dtype=torch.bfloat16, device=dev)
        _check(self.lib.ifx_moe_gather(_ptr(h), _ptr(row_pair), _ptr(rows), cap, top, width, _stream()), "moe_gather")
        act = torch.empty((cap, ff), dtype=torch.bfloat16, device=dev)
        if glu is not None:
            _check(self.lib.ifx_gemm_tcgen05_grouped_glu_offset(
                _ptr(rows), _ptr(w_up), _ptr(act), cap, ff, width, int(experts), _ptr(tile_group), ctypes.c_float(glu[0]),
                ctypes.c_float(glu[1]), ctypes.c_float(glu[2] if len(glu) > 2 else 1.0), _ptr(self.error_flag), _stream()),
                "moe experts (gate and up, tiles)")
        else:
            _check(self.lib.ifx_gemm_tcgen05_grouped(_ptr(rows), _ptr(w_up), _ptr(act), cap, ff, width, int(experts), ff,
                                                     _ptr(tile_group), _ptr(None), 2, _ptr(self.error_flag), _stream()),
                   "moe experts (up, tiles)")
        y = torch.empty((cap, width), dtype=torch.float32, device=dev)
        _check(self.lib.ifx_gemm_tcgen05_grouped(_ptr(act), _ptr(w_down), _ptr(y), cap, width, ff, int(experts), width,
                                                 _ptr(tile_group), _ptr(row_scale), 3, _ptr(self.error_flag), _stream()),
               "moe experts (down, tiles)")
        out = torch.empty((T, width), dtype=out_dtype, device=dev)
        _check(self.lib.ifx_moe_combine(_ptr(h), _ptr(y), _ptr(ids), _ptr(weights), _ptr(pair_row), _ptr(out), T, top,
                                        int(experts), width, _DT[out_dtype], _stream()), "moe_combine")
        self.launches += 5
        return out

    # ------------------------------------------- pairs of mixers, scans with a decayed matrix state
    def bigram_add(self, x, table, token_ids, state, mul_prev, mul_cur, buckets, vocab, ctx):
        """x[t] += table[(token before * mul_prev + token * mul_cur) mod buckets], the last row (`buckets`) at position 0;
        the token before a span's first one is state[slot, 0] (int32), which then takes the span's last token."""
        T, H = x.shape
        _need(x.dtype == torch.float32 and x.is_contiguous() and table.is_contiguous() and tuple(table.shape) == (buckets + 1, H)
              and state is not None and state.dtype == torch.int32, "bigram_add: bad operands")
        _check(self.lib.ifx_bigram_add(_ptr(x), _ptr(table), _ptr(token_ids), _ptr(ctx.positions), _ptr(ctx.token_req),
                                       _ptr(ctx.req_slot), _ptr(ctx.cu_seqlens), _ptr(state), ctypes.c_longlong(state.stride(0)),
                                       T, H, int(vocab), ctypes.c_longlong(mul_prev), ctypes.c_longlong(mul_cur), int(buckets),
                                       _DT[table.dtype], _stream()), "bigram_add")
        self.launches += 1

    def rmsnorm_pair(self, x, w_a, eps_a, w_b, eps_b, out_dtype, delta=None, vectors=None):
        """x += delta (if any); two RMS norms of the same float32 rows, one kernel.  `vectors` (a.s_a, b, s_b, b2 as in
        residual_add_vectors): x += s_a * a + s_b * (b + b2) in the same kernel."""
        if delta is not None:
            self.residual_add(x, delta)
        T, H = x.shape
        va = vb = vb2 = vsa = vsb = None
        if vectors is not None:
            va, vsa, vsb = self.materialize(vectors.a), vectors.s_a, vectors.s_b
            vb = None if vectors.b is None else self.materialize(vectors.b)
            vb2 = None if vectors.b2 is None else self.materialize(vectors.b2)
            if vb is not None and vb2 is not None and vb2.dtype != vb.dtype:
                vb2 = vb2.to(vb.dtype)
            _need(va.shape == x.shape and va.is_contiguous() and (vb is None or (vb.shape == x.shape and vb.is_contiguous()))
                  and (vb2 is None or (vb is not None and vb2.is_contiguous())), "rmsnorm_pair: the sum's rows do not fit")
        _need(x.dtype == torch.float32 and x.is_contiguous() and w_a.numel() == H and w_b.numel() == H
              and w_a.dtype == torch.float32 and w_b.dtype == torch.float32, "rmsnorm_pair: bad operands")
        out_a = torch.empty((T, H), dtype=out_dtype, device=x.device)
        out_b = torch.empty((T, H), dtype=out_dtype, device=x.device)
        _check(self.lib.ifx_rmsnorm_pair(_ptr(x), _ptr(w_a), ctypes.c_float(eps_a), _ptr(w_b), ctypes.c_float(eps_b), _ptr(out_a),
                                         _ptr(out_b), T, H, _DT[out_dtype], _ptr(va), _DT[va.dtype] if va is not None else 0,
                                         _ptr(vsa), _ptr(vb), _ptr(vb2), _DT[vb.dtype] if vb is not None else 0, _ptr(vsb),
                                         _stream()), "rmsnorm_pair")
        self.launches += 1
        return out_a, out_b

    def gate_mul(self, a, g, kind):
        """a * sigmoid(g) (`sigmoid`) or a * silu(g) (`silu`), in a's dtype."""
        _need(kind in ("sigmoid", "silu") and a.shape == g.shape and a.dtype == g.dtype and a.is_contiguous() and g.is_contiguous(),
              "gate_mul: bad operands")
        out = torch.empty_like(a)
        _check(self.lib.ifx_gate_mul(_ptr(a), _ptr(g), _ptr(out), ctypes.c_longlong(a.numel()), _DT[a.dtype], int(kind == "silu"),
                                     _stream()), "gate_mul")
        self.launches += 1
        return out

    @staticmethod
    def _rows_f32(t, what):
        _need(t.dtype == torch.float32 and t.dim() == 2 and t.stride(1) == 1, f"{what}: float32 rows with unit column stride")
        return ctypes.c_void_p(t.data_ptr()), ctypes.c_longlong(t.stride(0))

    def decay_scan(self, q, k, v, raw, state, ctx, heads, groups, dk, dv, decay, tau=1.0, q_scale=1.0, step_bias=None,
                   log_rate=None, skip=None):
        """Per request and head a float32 matrix S, kept in `state` [slots, >= heads dv dk] as [head, value channel, key
        channel]: S <- diag(w_t) S + k_t v_t^T, o_t = S^T (q_scale q_t) with the new S.  q, k: float32 [T, groups dk]
        (head h reads group h // (heads / groups)); v: [T, heads dv]; rows may be slices of wider rows.  Returns
        float32 [T, heads dv].
        decay `sigmoid_root`: raw [T, heads dk], w = sigmoid(raw)^(1/tau).
        decay `softplus_step`: raw [T, heads], dt = softplus(raw + step_bias), w = exp(-exp(log_rate) dt) for the whole
        head, k is multiplied by dt, and skip[h] v_t is added to o_t."""
        T = q.shape[0]
        _need(decay in ("sigmoid_root", "softplus_step"), f"decay_scan: unknown decay {decay!r}")
        mode = 0 if decay == "sigmoid_root" else 1
        _need(q.shape[1] == groups * dk and k.shape[1] == groups * dk and v.shape[1] == heads * dv
              and raw.shape[1] == (heads * dk if mode == 0 else heads) and k.shape[0] == T and v.shape[0] == T and raw.shape[0] == T,
              "decay_scan: the rows do not fit the head counts")
        _need(state is not None and state.dtype == torch.float32 and state.stride(1) == 1 and state.shape[1] >= heads * dv * dk,
              "decay_scan: the state does not fit the heads")
        for vec in (step_bias, log_rate, skip):
            _need(vec is None or (vec.dtype == torch.float32 and vec.numel() == heads and vec.is_contiguous()),
                  "decay_scan: per-head vectors are float32 [heads]")
        out = torch.empty((T, heads * dv), dtype=torch.float32, device=q.device)
        scratch = None                                     # steps with long spans make their decays in a pass of their own
        if ctx.max_span >= 64:
            scratch = torch.empty(T * (heads * dk if mode == 0 else 2 * heads), dtype=torch.float32, device=q.device)
        _check(self.lib.ifx_decay_scan(*self._rows_f32(q, "decay_scan q"), *self._rows_f32(k, "decay_scan k"),
                                       *self._rows_f32(v, "decay_scan v"), *self._rows_f32(raw, "decay_scan raw"), _ptr(state),
                                       ctypes.c_longlong(state.stride(0)), _ptr(ctx.req_slot), _ptr(ctx.cu_seqlens), _ptr(out),
                                       _ptr(step_bias), _ptr(log_rate), _ptr(skip), ctx.num_requests, T, int(ctx.max_span), int(heads),
                                       int(groups), int(dk), int(dv), mode, ctypes.c_float(tau), ctypes.c_float(q_scale), 296,
                                       _ptr(scratch), _stream()), "decay_scan")
        self.launches += 1 + int(scratch is not None)
        return out

    def gated_groupnorm(self, y, gate, w, eps, groups, gate_first, out_dtype):
        """Rows of y (float32 [T, C]) in `groups` equal parts, each over its own root mean square, times w (of size C, or
        of a part's size and then the same for every part) and silu(gate) (float32 rows, maybe a slice of wider ones):
        the gate multiplies before the norm (`gate_first`) or behind it."""
        T, C = y.shape
        _need(y.dtype == torch.float32 and y.is_contiguous() and tuple(gate.shape) == (T, C) and w.dtype == torch.float32
              and w.is_contiguous() and C % groups == 0 and w.numel() in (C, C // groups), "gated_groupnorm: bad operands")
        out = torch.empty((T, C), dtype=out_dtype, device=y.device)
        gp, gs = self._rows_f32(gate, "gated_groupnorm gate")
        _check(self.lib.ifx_gated_groupnorm(_ptr(y), gp, gs, _ptr(w), int(w.numel()), ctypes.c_float(eps), _ptr(out), T, C,
                                            int(groups), int(bool(gate_first)), _DT[out_dtype], _stream()), "gated_groupnorm")
        self.launches += 1
        return out

    def pair_combine(self, a, b, w_a, w_b, c_a, c_b, eps):
        """float32 [T, C]: c_a a + c_b b, or with weights c_a a / rms(a) * w_a + c_b b / rms(b) * w_b (a, b in any dtype)."""
        T, C = a.shape
        _need(a.is_contiguous() and b.is_contiguous() and a.shape == b.shape and (w_a is None) == (w_b is None),
              "pair_combine: rows of one shape")
        out = torch.empty((T, C), dtype=torch.float32, device=a.device)
        _check(self.lib.ifx_pair_combine(_ptr(a), _DT[a.dtype], _ptr(b), _DT[b.dtype], _ptr(w_a), _ptr(w_b), ctypes.c_float(c_a),
                                         ctypes.c_float(c_b), ctypes.c_float(eps), _ptr(out), T, C, _stream()), "pair_combine")
        self.launches += 1
        return out

    def residual_add_vectors(self, x, a, s_a, b=None, s_b=None, b2=None):
        """x += s_a * a + s_b * (b + b2), element by element along a row (a vector None: ones; b, b2 may be None)."""
        T, C = x.shape
        a = self.materialize(a)
        b = None if b is None else self.materialize(b)
        b2 = None if b2 is None else self.materialize(b2)
        if b is not None and b2 is not None and b2.dtype != b.dtype:
            b2 = b2.to(b.dtype)
        _need(x.dtype == torch.float32 and x.is_contiguous() and a.shape == x.shape and a.is_contiguous()
              and (b is None or (b.shape == x.shape and b.is_contiguous())) and (b2 is None or (b is not None and b2.is_contiguous())),
              "residual_add_vectors: bad operands")
        _check(self.lib.ifx_residual_add_vectors(_ptr(x), _ptr(a), _DT[a.dtype], _ptr(s_a), _ptr(b), _ptr(b2),
                                                 _DT[b.dtype] if b is not None else 0, _ptr(s_b), T, C, _stream()),
               "residual_add_vectors")
        self.launches += 1

    # ---------------------------------------------------------------- sampling
    def argmax(self, logits):
        R, V = logits.shape
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        if V >= 16384 and R <= 256:                      # long rows, few of them: many blocks per row
            _check(self.lib.ifx_argmax_chunks(_ptr(logits), _ptr(out), R, V, 32, _ptr(self._argmax_val),
                                              _ptr(self._argmax_idx), _ptr(self._argmax_tickets), _stream()), "argmax")
            self.launches += 1
            return out
        _check(self.lib.ifx_argmax(_ptr(logits), _ptr(out), R, V, _stream()), "argmax")
        self.launches += 1
        return out

    def penalties(self, logits, tokens, counts, rep, freq, pres):
        R, V = logits.shape
        _check(self.lib.ifx_penalties(_ptr(logits), _ptr(tokens), _ptr(counts), _ptr(rep), _ptr(freq), _ptr(pres),
                                      R, tokens.shape[1], V, _stream()), "penalties")
        self.launches += 1

    def logit_bias(self, logits, rows, tokens, bias):
        R, V = logits.shape
        _check(self.lib.ifx_logit_bias(_ptr(logits), _ptr(rows), _ptr(tokens), _ptr(bias), rows.numel(), R, V,
                                       _stream()), "logit_bias")
        self.launches += 1

    def sample(self, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, step, features=3):
        """One draw per row (see sampling.cu).  Rows are spread over many blocks; `features` says which
        filters any row uses (bit 0: top-k, bit 1: top-p) so that the passes of the others are not launched."""
        R, V = logits.shape
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        if R > self._sample_capacity:                    # the scratch's layout goes with its capacity
            self._sample_capacity = max(64, 1 << (R - 1).bit_length())
            self._sample_scratch = torch.zeros(int(self.lib.ifx_sample_scratch_bytes(self._sample_capacity)),
                                               dtype=torch.uint8, device=logits.device)
        passes = 3 + (1 if features & 3 else 0) + (2 if features & 1 else 0) + (3 if features & 2 else 0)
        _check(self.lib.ifx_sample_blocks(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p),
                                          _ptr(seed_lo), _ptr(seed_hi), _ptr(step), _ptr(out), R, V, int(features),
                                          _ptr(self._sample_scratch), self._sample_capacity, _stream()), "sample")
        self.launches += passes
        return out

    def sample_one_block(self, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, step):
        """The same draw with one block per row and thresholds by bisection (kept for comparison)."""
        R, V = logits.shape
        probs = torch.empty((R, V), dtype=torch.float32, device=logits.device)
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        _check(self.lib.ifx_sample(_ptr(logits), _ptr(probs), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                   _ptr(min_p), _ptr(seed_lo), _ptr(seed_hi), _ptr(step), _ptr(out), R, V,
                                   _stream()), "sample")
        self.launches += 1
        return out
