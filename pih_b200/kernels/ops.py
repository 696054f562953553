"""``CudaOps``: the calls that parts make, bound to the kernel pack through ctypes.

Every method launches hand-written kernels from ``csrc/`` on the current
CUDA stream.  Matrix products in bfloat16 go to the library (cuBLAS through
``torch.mm``) where the reference does the same
(src/backend/cuda/gemm_plan.cpp:192-197 runs every product through
cuBLASLt); in float32 they run on the pack's own FMA kernel so that no
reduced-precision mode can slip in.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

_DT = {torch.float32: 0, torch.bfloat16: 1}
_ERRORS = {1: "a token id is outside the vocabulary", 2: "a row maps to no cache page",
           3: "logits contain a non-finite value", 4: "a position is outside the rotation table",
           5: "attention softmax denominator is not positive and finite", 6: "a device wait timed out"}

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


class KernelError(RuntimeError):
    pass


def error_text(code: int) -> str:
    """What a value of the device's error word means."""
    return _ERRORS.get(code, f"error code {code}")


class CudaOps:
    def __init__(self, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("pih_b200 runs on a CUDA device only (there is no CPU path), "
                               "and torch.cuda.is_available() is False")
        self.device = torch.device(device if device is not None else "cuda:0")
        if self.device.type != "cuda":
            raise RuntimeError(f"pih_b200 runs on a CUDA device only, got {self.device}")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise RuntimeError(f"the kernel pack is built for sm_100a; this device is sm_{major}{minor}")
        path = build.library_path()
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise RuntimeError(f"pih_b200: the kernel pack {path} could not be loaded: {e}") from None
        self.library_path = path
        # library products must accumulate in 32-bit all the way: no bf16 partial sums in split-K
        # reductions, no TF32
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        torch.backends.cuda.matmul.allow_tf32 = False
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._error = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0
        self._attn_scratch = None          # partials of the split-KV attention kernel, grown on demand
        self._retired_scratch = []
        self._kv_maps = {}                 # cache tensor (address, shape) -> 128-byte TMA descriptor
        self.tma_attention = True          # False: the split kernel gathers with cp.async instead of TMA
        self.tcgen05_attention = True      # False: prompt portions use the mma.sync tile kernel
        self.fused_qk_attention = True     # decode-only steps: q/k norm, rotation and cache append inside the attention kernel
        self.fused_qk_max_requests = 32    # ... up to this batch (measured: 16 requests +4 %, 32 even, 64 -1.6 %)
        self.cluster_attention = True      # False: splits always merge through scratch memory and tickets
        self.attention_split = 0           # keys per split of the decode attention kernel; 0: from the context, on the device
        self.tensor_core_attention = True  # False: bf16 attention runs on the generic kernel too
        self._tcgen05_swiglu_min_rows = 1536     # the library's default (see the property)
        self.tcgen05_min_rows = None       # bf16 products with at least this many rows use the pack's tcgen05 kernel
        self.skinny_max_rows = 16          # bf16 products with at most this many rows use the fused few-rows kernel
        self.fused_residual = True         # ... and add the residual in the epilogue of output projections
        self.native_blocks = True          # blocks of the built-in parts are issued by one native call each
        self._native = None
        self._declare()

    @property
    def tcgen05_swiglu_min_rows(self):
        """Prompt portions of at least this many rows run their gate/up product on the pack's tcgen05 kernel on
        pairs of SMs with SiLU-mul in its epilogue, when its tiles fill the SM pairs well (see
        pih_pair_swiglu_wanted); None: never.  The setting is the library's: native blocks follow it."""
        return self._tcgen05_swiglu_min_rows

    @tcgen05_swiglu_min_rows.setter
    def tcgen05_swiglu_min_rows(self, rows) -> None:
        self.set_pair_swiglu_rule(rows)

    def set_pair_swiglu_rule(self, min_rows, min_fill_percent: int = -1) -> None:
        """``min_rows`` as ``tcgen05_swiglu_min_rows``; ``min_fill_percent``: how full the tiles must make the
        rounds of SM pairs (80 by default; 0 sends every shape of enough rows to that kernel; -1: unchanged)."""
        self._tcgen05_swiglu_min_rows = min_rows
        self.lib.pih_set_pair_swiglu_rule(int(min_rows) if min_rows else 0, int(min_fill_percent))

    # -- plumbing ---------------------------------------------------------------
    def _declare(self) -> None:
        lib = self.lib
        for name in ("pih_embedding", "pih_rmsnorm", "pih_qk_norm_rope_kv_write", "pih_silu_mul",
                     "pih_gather_rows", "pih_gemm_simt", "pih_paged_attention_generic", "pih_argmax",
                     "pih_sample", "pih_selected_logprob", "pih_top_logprobs", "pih_paged_attention_mma", "pih_gemm_tcgen05", "pih_make_kv_tensor_map",
                     "pih_attention_prefill_tcgen05", "pih_gemm_skinny", "pih_set_dependent_launch", "pih_set_attention_cluster_merge",
                     "pih_gemm_skinny_f32out",
                     "pih_qk_attention_fused", "pih_gemm_tcgen05_pair", "pih_set_attention_side_by_side", "pih_set_skinny_rule",
                     "pih_gemm_simt_batched", "pih_embedding_stream", "pih_rmsnorm_stream", "pih_causal_conv",
                     "pih_gated_delta_rule", "pih_gated_rmsnorm", "pih_rglru_scan", "pih_latent_write",
                     "pih_latent_attention_generic", "pih_moe_route", "pih_moe_experts", "pih_moe_combine_bf16", "pih_latent_attention_split", "pih_latent_attention_splits", "pih_latent_attention_mma", "pih_batched_gemv",
                     "pih_stream_cast", "pih_stream_norm_add", "pih_bias_xielu", "pih_add_gated", "pih_retention",
                     "pih_diff_qk_prepare", "pih_diff_attention", "pih_diff_attention_tile_takes", "pih_moe_route_scored",
                     "pih_act_mul", "pih_embed_positions", "pih_hyper_stream", "pih_window_qk_prepare",
                     "pih_window_attention", "pih_window_attention_tile_takes", "pih_embed_bigram", "pih_rmsnorm_rows",
                     "pih_rotate_heads", "pih_gate_mul", "pih_unary_act", "pih_scale_rows", "pih_moe_gather_scaled"):
            getattr(lib, name).restype = c_int
        lib.pih_attention_scratch_floats.restype = c_ll
        lib.pih_top_logprobs_scratch_words.restype = c_ll
        lib.pih_moe_route_words.restype = c_ll

    def _native_supports(self, block) -> bool:
        from .native_block import NativeBlocks
        return NativeBlocks.supports(block)

    def native_block(self, block, h, delta, step, cache):
        """A pre-norm block of the built-in parts through one native call (``native_block.NativeBlocks``); None when
        that path is off or does not take the block."""
        if not self.native_blocks:
            return None
        if self._native is None:
            from .native_block import NativeBlocks
            self._native = NativeBlocks(self)
        return self._native.run(block, h, delta, step, cache)

    def set_dependent_launch(self, on: bool) -> bool:
        """Whether the pack's kernels are launched so that each may begin while the one before it drains
        (programmatic dependent launch; the default).  Returns the previous setting.  The setting is the
        library's, not this object's; CUDA graphs keep the setting they were captured under."""
        return bool(self.lib.pih_set_dependent_launch(1 if on else 0))

    def set_skinny_rule(self, on: bool) -> bool:
        """Whether the few-rows product declines the shapes for which the library's product with the separate
        kernels is faster (the default) or takes every shape it can.  Returns the previous setting (the library's)."""
        return bool(self.lib.pih_set_skinny_rule(1 if on else 0))

    def set_attention_side_by_side(self, on: bool) -> bool:
        """Whether, in a step with prompt portions and decoding requests, native blocks run the two attention
        kernels side by side — the decoding requests' in a stream that forks behind the q/k kernel and joins before
        the output projection (the default) — or one after the other.  Returns the previous setting; the setting is
        the library's, and CUDA graphs keep the one they were captured under."""
        return bool(self.lib.pih_set_attention_side_by_side(1 if on else 0))

    def set_attention_cluster_merge(self, on):
        """Whether 2 to 8 splits of one (request, kv head) of the decode attention run as a thread-block
        cluster that merges through distributed shared memory (True, the default: small partials are sent to
        the block that finishes them, larger ones fetched by it; "fetched": always fetched) or through scratch
        memory and tickets (False).  Returns the previous setting; the setting is the library's."""
        self.cluster_attention = bool(on)
        before = self.lib.pih_set_attention_cluster_merge(2 if on == "fetched" else 1 if on else 0)
        return "fetched" if before == 2 else bool(before)

    def _stream(self):
        # the raw handle of the current stream (torch.cuda.current_stream builds a Stream object: 8 us a call,
        # four milliseconds over the launches of an uncaptured step)
        return c_void_p(torch._C._cuda_getCurrentRawStream(self._device_index))

    def _check(self, rc: int, what: str) -> None:
        self.launches += 1
        if rc == 0:
            return
        if rc == -1:
            raise KernelError(f"{what}: bad argument")
        if rc == -2:
            raise KernelError(f"{what}: this size is not supported by the kernel")
        raise KernelError(f"{what}: CUDA error {rc}")

    @property
    def error_word(self) -> torch.Tensor:
        """int32 [1] on the device: 0, or the code of the first fault that a kernel reported since it was cleared."""
        return self._error

    def clear_errors(self) -> None:
        """Zero the error word (queued on the current stream, behind the kernels already queued there)."""
        self._error.zero_()

    def check_errors(self) -> None:
        """Read the device error word (synchronises); raise if a kernel reported something."""
        code = int(self._error.item())
        if code:
            self.clear_errors()
            raise KernelError(f"a kernel reported: {error_text(code)}")

    def _err(self):
        return c_void_p(self._error.data_ptr())

    # -- ops ----------------------------------------------------------------------
    def embedding(self, table: torch.Tensor, ids: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        rows, (vocab, hidden) = ids.shape[0], table.shape
        if out_dtype is not None and out_dtype != table.dtype:
            if out_dtype != torch.float32:
                raise ValueError("an embedding widens to float32 only")
            out = torch.empty(rows, hidden, dtype=torch.float32, device=table.device)      # a 32-bit residual stream
            rc = self.lib.pih_embedding_stream(_DT[table.dtype], _ptr(table), _ptr(ids), _ptr(out), rows, hidden, vocab,
                                               self._err(), self._stream())
            self._check(rc, "embedding_stream")
            return out
        out = torch.empty(rows, hidden, dtype=table.dtype, device=table.device)
        rc = self.lib.pih_embedding(_DT[table.dtype], _ptr(table), _ptr(ids), _ptr(out), rows, hidden, vocab,
                                    self._err(), self._stream())
        self._check(rc, "embedding")
        return out

    def rmsnorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, delta: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        width = x.shape[-1]
        assert x.is_contiguous() and (delta is None or (delta.is_contiguous() and delta.shape == x.shape))
        n_out = x.numel() // width if rows is None else rows.shape[0]
        out = torch.empty((n_out, width) if rows is not None else x.shape, dtype=x.dtype, device=x.device)
        rc = self.lib.pih_rmsnorm(_DT[x.dtype], _DT[weight.dtype], _ptr(x), _ptr(delta), _ptr(weight), _ptr(out),
                                  _ptr(rows), n_out, width, c_float(eps), self._stream())
        self._check(rc, "rmsnorm")
        return out

    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``x [M,K] . w [N,K]^T -> [M,N]``; fp32 accumulation; the output is
        rounded once to ``out_dtype`` (default: the dtype of ``x``)."""
        M, K = x.shape
        N = w.shape[0]
        out_dtype = out_dtype or x.dtype
        assert w.shape[1] == K and x.dtype == w.dtype and x.stride(1) == 1 and w.stride(1) == 1
        if x.dtype == torch.float32:
            out = torch.empty(M, N, dtype=torch.float32, device=x.device)
            rc = self.lib.pih_gemm_simt(0, 0, _ptr(x), _ptr(w), _ptr(out), M, N, K, c_ll(x.stride(0)),
                                        c_ll(w.stride(0)), c_ll(N), self._stream())
            self._check(rc, "gemm_simt")
            return out
        if out_dtype == torch.bfloat16 and M <= self.skinny_max_rows:
            out = self.linear_skinny(x, w)
            if out is not None:
                return out
        if out_dtype == torch.float32 and M <= self.skinny_max_rows and K % 32 == 0:
            out = torch.empty(M, N, dtype=torch.float32, device=x.device)
            rc = self.lib.pih_gemm_skinny_f32out(_ptr(x), _ptr(w), _ptr(out), M, N, K, c_ll(x.stride(0)),
                                                 c_ll(w.stride(0)), c_ll(N), self._err(), self._stream())
            if rc != -2:
                self._check(rc, "gemm_skinny_f32out")
                return out
        if self.tcgen05_min_rows is not None and M >= self.tcgen05_min_rows:
            out = self.linear_tcgen05(x, w, out_dtype)
            if out is not None:
                return out
        if out_dtype == torch.float32:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.mm(x, w.t())

    def linear_skinny(self, x: torch.Tensor, w: torch.Tensor, *, delta=None, norm_weight=None, eps: float = 0.0,
                      swiglu: bool = False, residual: Optional[torch.Tensor] = None, activation: str = "silu"):
        """The few-rows product (bf16, at most 16 rows) with its optional fused residual add, RMSNorm and
        SwiGLU (``activation`` "gelu_tanh": GELU in SiLU's place) in front and behind.  ``activation`` "relu2" without
        ``swiglu``: the output is the square of ``max(round(x . w^T), 0)`` (a two-matrix feed-forward's first half).
        ``residual``: the result is ``round(round(x . w^T) + residual)``.  Returns
        ``out`` — or ``(x + delta, out)`` when ``delta`` is given — or None when the kernel does not take the shape."""
        M, K = x.shape
        N = w.shape[0]
        if (x.dtype != torch.bfloat16 or M > 16 or K % 32 or K > 16384 or x.stride(1) != 1 or w.stride(1) != 1
                or (swiglu and (N % 16 or residual is not None)) or (not swiglu and activation == "relu2" and residual is not None)
                or (residual is not None and (residual.shape != (M, N) or not residual.is_contiguous()))):
            return None
        out = torch.empty(M, N // 2 if swiglu else N, dtype=torch.bfloat16, device=x.device)
        x_out = torch.empty_like(x) if delta is not None else None
        nd = _DT[norm_weight.dtype] if norm_weight is not None else 0
        rc = self.lib.pih_gemm_skinny(_ptr(x), _ptr(delta), _ptr(x_out), nd, _ptr(norm_weight), c_float(eps), _ptr(w),
                                      _ptr(out), _ptr(residual), M, N, K, c_ll(x.stride(0)), c_ll(w.stride(0)),
                                      c_ll(out.stride(0)),
                                      (2 if activation == "gelu_tanh" else 1) if swiglu else (3 if activation == "relu2" else 0),
                                      self._err(), self._stream())
        if rc == -2:
            return None
        self._check(rc, "gemm_skinny")
        return out if delta is None else (x_out, out)

    def linear_add(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor):
        """``round(round(x . w^T) + residual)`` as one kernel — an output projection with the residual add that
        follows it — or None when only the separate kernels can do it (the caller then passes the product on and
        the next norm adds it)."""
        if x.shape[0] > self.skinny_max_rows or not self.fused_residual:
            return None
        return self.linear_skinny(x, w, residual=residual)

    def linear_tcgen05_swiglu(self, x: torch.Tensor, w: torch.Tensor):
        """``SwiGLU(x . w^T)`` with the pack's tcgen05 product on pairs of SMs and SiLU-mul in its epilogue: ``w``
        holds blocks of 8 gate rows followed by their 8 up rows; returns ``[M, N / 2]`` (bf16), or None for shapes
        that the kernel does not take."""
        M, K = x.shape
        N = w.shape[0]
        if x.dtype != torch.bfloat16 or N % 16 or x.stride(1) != 1 or w.stride(1) != 1:
            return None
        out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=x.device)
        rc = self.lib.pih_gemm_tcgen05_pair(_DT[torch.bfloat16], _ptr(x), _ptr(w), _ptr(out), M, N, K,
                                            c_ll(x.stride(0)), c_ll(w.stride(0)), c_ll(out.stride(0)), 0, 1,
                                            self._err(), self._stream())
        if rc == -2:
            return None
        self._check(rc, "gemm_tcgen05_pair")
        return out

    def norm_linear(self, h: torch.Tensor, delta: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                    w: torch.Tensor, swiglu_interleave: int = 0):
        """``h' = h + delta`` (when delta is given), ``out = rmsnorm(h') . w^T`` and, with
        ``swiglu_interleave``, SiLU-mul over gate/up column blocks of that size.  Returns ``(h', out)``;
        ``h'`` may be ``h`` updated in place or a new tensor.  One kernel for few rows, else the separate ones."""
        if h.dtype == torch.bfloat16 and h.shape[0] <= self.skinny_max_rows and swiglu_interleave in (0, 8):
            if delta is not None:
                res = self.linear_skinny(h, w, delta=delta, norm_weight=norm_weight, eps=eps,
                                         swiglu=swiglu_interleave == 8)
                if res is not None:
                    return res
            else:
                out = self.linear_skinny(h, w, norm_weight=norm_weight, eps=eps, swiglu=swiglu_interleave == 8)
                if out is not None:
                    return h, out
        xn = self.rmsnorm(h, norm_weight, eps, delta=delta)
        if (swiglu_interleave == 8 and xn.dtype == torch.bfloat16
                and self.lib.pih_pair_swiglu_wanted(xn.shape[0], w.shape[0])):
            out = self.linear_tcgen05_swiglu(xn, w)
            if out is not None:
                return h, out
        out = self.linear(xn, w)
        if swiglu_interleave:
            out = self.silu_mul(out, swiglu_interleave)
        return h, out

    def linear_tcgen05(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                       tile_n: int = 0, pairs: bool = False):
        """The pack's tcgen05 / TMA product (bf16 in, fp32 accumulation).  Returns None when the
        operands cannot be described to TMA (K or a row stride not a multiple of 8).  ``pairs``: the kernel
        that puts two SMs on a 256-row tile (``tile_n`` 128 or 256)."""
        M, K = x.shape
        N = w.shape[0]
        out_dtype = out_dtype or x.dtype
        out = torch.empty(M, N, dtype=out_dtype, device=x.device)
        if pairs:
            rc = self.lib.pih_gemm_tcgen05_pair(_DT[out_dtype], _ptr(x), _ptr(w), _ptr(out), M, N, K,
                                                c_ll(x.stride(0)), c_ll(w.stride(0)), c_ll(N), tile_n, 0,
                                                self._err(), self._stream())
        else:
            rc = self.lib.pih_gemm_tcgen05(_DT[out_dtype], _ptr(x), _ptr(w), _ptr(out), M, N, K, c_ll(x.stride(0)),
                                           c_ll(w.stride(0)), c_ll(N), tile_n, self._err(), self._stream())
        if rc == -2:
            return None
        self._check(rc, "gemm_tcgen05")
        return out

    def linear_plain(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """The pack's FMA product for any supported dtype (plain twin of the tensor-core products)."""
        M, K = x.shape
        N = w.shape[0]
        out_dtype = out_dtype or x.dtype
        out = torch.empty(M, N, dtype=out_dtype, device=x.device)
        rc = self.lib.pih_gemm_simt(_DT[x.dtype], _DT[out_dtype], _ptr(x), _ptr(w), _ptr(out), M, N, K,
                                    c_ll(x.stride(0)), c_ll(w.stride(0)), c_ll(N), self._stream())
        self._check(rc, "gemm_simt")
        return out

    def qk_norm_rope_kv_write(self, qkv, *, heads, kv_heads, head_dim, q_norm, k_norm, eps, rope_table,
                              rotary_dim, positions, slot_mapping, kv_cache, write_kv) -> None:
        """Per-head RMSNorm and rotation of the q and k heads of the rows ``[q | k | v]``; q is changed in place,
        and with ``write_kv`` k and v go to their slots of the cache.  The k part of the rows is not to be read
        afterwards: it holds the new k only where the kernel also wrote it there (few rows, rows without a slot)."""
        rows = qkv.shape[0]
        wd = _DT[q_norm.dtype] if q_norm is not None else _DT[qkv.dtype]
        num_pages, page_size = kv_cache.shape[0], kv_cache.shape[3]
        max_pos = rope_table.shape[0] if rope_table is not None else 0
        rc = self.lib.pih_qk_norm_rope_kv_write(
            _DT[qkv.dtype], wd, _ptr(qkv), qkv.stride(0), rows, heads, kv_heads, head_dim, _ptr(q_norm),
            _ptr(k_norm), c_float(eps), _ptr(rope_table), rotary_dim, max_pos, _ptr(positions),
            _ptr(slot_mapping), _ptr(kv_cache), page_size, num_pages, 1 if write_kv else 0, self._err(),
            self._stream())
        self._check(rc, "qk_norm_rope_kv_write")

    def paged_attention(self, qkv, *, heads, kv_heads, head_dim, kv_cache, block_table, step, scale,
                        window) -> torch.Tensor:
        """Attention of the step's rows over the cache.  bf16 runs on the tensor-core kernels
        when they have an instance for ``head_dim``; everything else on the generic kernel."""
        if self.tensor_core_attention and qkv.dtype == torch.bfloat16 and head_dim in self.MMA_HEAD_DIMS:
            return self.paged_attention_mma(qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                            kv_cache=kv_cache, block_table=block_table, step=step,
                                            scale=scale, window=window)
        return self.paged_attention_generic(qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                            kv_cache=kv_cache, block_table=block_table,
                                            request_of_row=step.request_of_row, positions=step.positions,
                                            scale=scale, window=window)

    MMA_HEAD_DIMS = (16, 32, 64, 80, 96, 128, 256)

    @staticmethod
    def attention_plan(host_cu_q, host_q_start, group: int):
        """(tile_max_q, dec_tok_cap, dec_max_ctx): a request is decode-like when it brings at most
        16 packed rows (rows * heads / kv_heads)."""
        tile_max_q = dec_cap = dec_ctx = 0
        for r in range(len(host_q_start)):
            n = host_cu_q[r + 1] - host_cu_q[r]
            if n * group <= 16:
                dec_cap = max(dec_cap, n)
                dec_ctx = max(dec_ctx, host_q_start[r] + n)
            else:
                tile_max_q = max(tile_max_q, n)
        return tile_max_q, dec_cap, dec_ctx

    def splits_for(self, num_requests: int, kv_heads: int, max_ctx: int = 0) -> int:
        """Splits per request of the decode attention: as many as fill the 2 x 148 CTA slots of the GPU in
        one wave (small batches are cut finely so that enough CTAs pull bandwidth, large ones not at all).
        Up to eight splits merge as a thread-block cluster, which is what a short context wants (the merge
        is most of its time); a long context wants every slot pulling (one request of 32768 keys: 69 us with
        8 splits, 34 us with 37), so beyond ``CLUSTER_MAX_KEYS`` keys per split the finer cut with the merge
        through scratch memory is taken.  A function of the batch size and the longest context that the
        step's block tables can hold, not of the contexts themselves: a captured step keeps its grid."""
        slots = (2 * 148) // max(1, num_requests * kv_heads)
        if self.cluster_attention and self.tma_attention and slots > 8 and max_ctx <= 8 * self.CLUSTER_MAX_KEYS:
            return 8                                   # one portable cluster per (request, kv head)
        return max(1, min(64, slots))

    CLUSTER_MAX_KEYS = 768

    def reserve_attention_scratch(self, num_requests, dec_tok_cap, heads, kv_heads, head_dim, max_ctx) -> None:
        """Make the split kernel's scratch large enough (before a CUDA graph that uses it is
        captured: an allocation cannot happen under capture).  A buffer that is outgrown is kept
        alive, because captured graphs hold its address."""
        splits = (-(-max_ctx // self.attention_split) if self.attention_split
                  else self.splits_for(num_requests, kv_heads, max_ctx))
        need = self.lib.pih_attention_scratch_floats(num_requests, dec_tok_cap, heads, kv_heads, head_dim, splits)
        if self._attn_scratch is None or self._attn_scratch.numel() < need:
            if self._attn_scratch is not None:
                self._retired_scratch.append(self._attn_scratch)     # captured graphs may still point at it
            # zeroed: the leading words are the kernel's tickets, which it leaves at zero
            self._attn_scratch = torch.zeros(int(need * 1.25) + 1024, dtype=torch.float32, device=self.device)

    def kv_tensor_map(self, kv_cache: torch.Tensor):
        """The TMA descriptor of one schedule entry's cache, made once; None when TMA cannot describe it."""
        key = (kv_cache.data_ptr(), tuple(kv_cache.shape))
        if key not in self._kv_maps:
            buf = ctypes.create_string_buffer(128)
            num_pages, _, kv_heads, page_size, head_dim = kv_cache.shape
            rc = self.lib.pih_make_kv_tensor_map(buf, _ptr(kv_cache), c_ll(num_pages), kv_heads, page_size, head_dim)
            self._kv_maps[key] = buf if rc == 0 else None
        return self._kv_maps[key]

    def paged_attention_mma(self, qkv, *, heads, kv_heads, head_dim, kv_cache, block_table, step, scale,
                            window, plan=None) -> torch.Tensor:
        rows = qkv.shape[0]
        group = heads // kv_heads
        plans = getattr(step, "attention_plans", None)
        if plan is None and plans is not None and group in plans:
            plan = plans[group]
        if plan is None:
            plan = self.attention_plan(step.host_cu_q, step.host_q_start, group)
            if plans is not None:
                plans[group] = plan
        tile_max_q, dec_cap, dec_ctx = plan
        out = torch.empty(rows, heads * head_dim, dtype=qkv.dtype, device=qkv.device)
        num_pages, page_size = kv_cache.shape[0], kv_cache.shape[3]
        split = self.attention_split                       # 0: cut on the device into `nsplits` parts
        nsplits = self.splits_for(step.num_requests, kv_heads, dec_ctx)
        max_ctx_ptr = getattr(step, "meta", None)
        if split == 0 and max_ctx_ptr is None:              # a caller without a packed batch: fix the cut here
            split = max(64, -(-(-(-max(dec_ctx, 1) // nsplits)) // 64) * 64)
        scratch = None
        if dec_cap > 0:
            self.reserve_attention_scratch(step.num_requests, dec_cap, heads, kv_heads, head_dim, dec_ctx)
            scratch = self._attn_scratch
        kv_map = self.kv_tensor_map(kv_cache) if (self.tma_attention or self.tcgen05_attention) else None
        if tile_max_q > 0 and self.tcgen05_attention and kv_map is not None and head_dim in (64, 128) \
                and page_size in (8, 16, 32, 64):
            rc = self.lib.pih_attention_prefill_tcgen05(
                _ptr(qkv), qkv.stride(0), rows, _ptr(out), _ptr(block_table), block_table.shape[1], _ptr(step.cu_q),
                _ptr(step.q_start), step.num_requests, tile_max_q, heads, kv_heads, head_dim, page_size, num_pages,
                c_float(scale), int(window), kv_map, self._err(), self._stream())
            self._check(rc, "attention_prefill_tcgen05")
            tile_max_q = 0                                  # done; what is left is decode-like
            if dec_cap == 0:
                return out
        rc = self.lib.pih_paged_attention_mma(
            _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(kv_cache), _ptr(block_table), block_table.shape[1],
            _ptr(step.cu_q), _ptr(step.q_start), rows, step.num_requests, tile_max_q, dec_cap, dec_ctx, heads, kv_heads, head_dim, page_size, num_pages,
            c_float(scale), int(window), split, nsplits, _ptr(max_ctx_ptr), _ptr(scratch),
            kv_map if (self.tma_attention and dec_cap > 0) else None,
            self._err(), self._stream())
        self._check(rc, "paged_attention_mma")
        return out

    def qk_attention_fused(self, qkv, *, heads, kv_heads, head_dim, q_norm, k_norm, eps, rope_table, rotary_dim,
                           kv_cache, block_table, step, scale, window, write_kv):
        """``qk_norm_rope_kv_write`` and ``paged_attention`` as one kernel, for steps whose requests are all
        decode-like (bf16, the TMA split kernel's shapes, rotation over the whole head).  ``qkv`` stays raw.
        Returns the attention output, or None when the separate kernels have to run."""
        if (not self.fused_qk_attention or qkv.dtype != torch.bfloat16 or not self.tensor_core_attention
                or not self.tma_attention or (rope_table is not None and rotary_dim != head_dim)
                or (q_norm is not None and k_norm is not None and q_norm.dtype != k_norm.dtype)):
            return None
        group = heads // kv_heads
        plans = getattr(step, "attention_plans", None)
        plan = plans[group] if plans is not None and group in plans else None
        if plan is None:
            plan = self.attention_plan(step.host_cu_q, step.host_q_start, group)
            if plans is not None:
                plans[group] = plan
        tile_max_q, dec_cap, dec_ctx = plan
        max_ctx_ptr = getattr(step, "meta", None)
        if (tile_max_q > 0 or dec_cap <= 0 or (self.attention_split == 0 and max_ctx_ptr is None)
                or step.num_requests > self.fused_qk_max_requests):
            return None
        kv_map = self.kv_tensor_map(kv_cache)
        if kv_map is None:
            return None
        rows = qkv.shape[0]
        num_pages, page_size = kv_cache.shape[0], kv_cache.shape[3]
        nsplits = self.splits_for(step.num_requests, kv_heads, dec_ctx)
        self.reserve_attention_scratch(step.num_requests, dec_cap, heads, kv_heads, head_dim, dec_ctx)
        out = torch.empty(rows, heads * head_dim, dtype=qkv.dtype, device=qkv.device)
        norm = q_norm if q_norm is not None else k_norm
        rc = self.lib.pih_qk_attention_fused(
            _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(kv_cache), _ptr(block_table), block_table.shape[1],
            _ptr(step.cu_q), _ptr(step.q_start), rows, step.num_requests, dec_cap, dec_ctx, heads, kv_heads, head_dim,
            page_size, num_pages, c_float(scale), int(window), self.attention_split, nsplits, _ptr(max_ctx_ptr),
            _ptr(self._attn_scratch), kv_map, _DT[norm.dtype] if norm is not None else 1, _ptr(q_norm), _ptr(k_norm),
            c_float(eps), _ptr(rope_table), rope_table.shape[0] if rope_table is not None else 0,
            1 if write_kv else 0, self._err(), self._stream())
        if rc == -2:
            return None
        self._check(rc, "qk_attention_fused")
        return out

    def paged_attention_generic(self, qkv, *, heads, kv_heads, head_dim, kv_cache, block_table,
                                request_of_row, positions, scale, window) -> torch.Tensor:
        rows = qkv.shape[0]
        out = torch.empty(rows, heads * head_dim, dtype=qkv.dtype, device=qkv.device)
        num_pages, page_size = kv_cache.shape[0], kv_cache.shape[3]
        rc = self.lib.pih_paged_attention_generic(
            _DT[qkv.dtype], _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(kv_cache), _ptr(block_table),
            block_table.shape[1], _ptr(request_of_row), _ptr(positions), rows, heads, kv_heads, head_dim,
            page_size, num_pages, c_float(scale), int(window), self._err(), self._stream())
        self._check(rc, "paged_attention_generic")
        return out

    def gather_rows(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """``x[rows]`` for contiguous x ``[n, width]`` and int32 ``rows``."""
        assert x.is_contiguous() and rows.dtype == torch.int32
        out = torch.empty(rows.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
        rc = self.lib.pih_gather_rows(_DT[x.dtype], _ptr(x), _ptr(rows), _ptr(out), rows.shape[0], x.shape[1], self._stream())
        self._check(rc, "gather_rows")
        return out

    def act_mul(self, gate_up: torch.Tensor, interleave: Optional[int] = None, activation: str = "silu") -> torch.Tensor:
        """``act(g) * u`` with ``activation`` "silu" or "gelu_tanh" (``g / 2 (1 + tanh(sqrt(2 / pi) (g + 0.044715
        g^3)))``), in 32-bit, rounded once; columns as for ``silu_mul``."""
        rows, two_i = gate_up.shape
        inter = two_i // 2
        out = torch.empty(rows, inter, dtype=gate_up.dtype, device=gate_up.device)
        rc = self.lib.pih_act_mul(_DT[gate_up.dtype], {"silu": 0, "gelu_tanh": 1}[activation], _ptr(gate_up), _ptr(out),
                                  c_ll(rows), inter, interleave if interleave is not None else inter, self._stream())
        self._check(rc, "act_mul")
        return out

    def silu_mul(self, gate_up: torch.Tensor, interleave: Optional[int] = None) -> torch.Tensor:
        """``silu(g) * u``; the columns of ``gate_up`` come in blocks of ``interleave`` gate columns
        followed by their up columns (default: all gates, then all ups)."""
        rows, two_i = gate_up.shape
        inter = two_i // 2
        out = torch.empty(rows, inter, dtype=gate_up.dtype, device=gate_up.device)
        rc = self.lib.pih_silu_mul(_DT[gate_up.dtype], _ptr(gate_up), _ptr(out), c_ll(rows), inter,
                                   interleave or inter, self._stream())
        self._check(rc, "silu_mul")
        return out

    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        rows, vocab = logits.shape
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        scratch = torch.empty(rows * 128, dtype=torch.float32, device=logits.device) if vocab >= 8192 else None
        rc = self.lib.pih_argmax(_ptr(logits), rows, vocab, _ptr(out), _ptr(scratch), self._err(), self._stream())
        self._check(rc, "argmax")
        return out

    def selected_logprob(self, logits: torch.Tensor, tokens: torch.Tensor, fparams: Optional[torch.Tensor] = None,
                         iparams: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The log-probability of ``tokens[row]`` under each row's scaled logits (fp32 ``[rows]``); the
        parameters are those given to ``sample``, or none for greedy rows."""
        rows, vocab = logits.shape
        out = torch.empty(rows, dtype=torch.float32, device=logits.device)
        rc = self.lib.pih_selected_logprob(_ptr(logits), rows, vocab, _ptr(tokens), _ptr(fparams), _ptr(iparams),
                                           iparams.shape[1] if iparams is not None else 0, _ptr(out), self._err(),
                                           self._stream())
        self._check(rc, "selected_logprob")
        return out

    def top_logprobs(self, logits: torch.Tensor, count: int, fparams: Optional[torch.Tensor] = None,
                     iparams: Optional[torch.Tensor] = None):
        """The ``count`` (1 to 20) most probable ids of every row that are not suppressed — by value, then by id —
        and their log-probabilities under the row's scaled logits: ``(int32 [rows, count], fp32 [rows, count])``;
        the parameters are those given to ``sample``, or none for greedy rows."""
        rows, vocab = logits.shape
        words = self.lib.pih_top_logprobs_scratch_words(rows, vocab, count)
        if words < 0:
            raise ValueError(f"top_logprobs takes no vocabulary of {vocab}")
        scratch = torch.empty(max(int(words), 1), dtype=torch.float32, device=logits.device)
        ids = torch.empty(rows, count, dtype=torch.int32, device=logits.device)
        lps = torch.empty(rows, count, dtype=torch.float32, device=logits.device)
        rc = self.lib.pih_top_logprobs(_ptr(logits), rows, vocab, count, _ptr(fparams), _ptr(iparams),
                                       iparams.shape[1] if iparams is not None else 0, _ptr(ids), _ptr(lps),
                                       _ptr(scratch), self._err(), self._stream())
        self._check(rc, "top_logprobs")
        return ids, lps

    def sample(self, logits: torch.Tensor, fparams: torch.Tensor, iparams: torch.Tensor) -> torch.Tensor:
        rows, vocab = logits.shape
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        rc = self.lib.pih_sample(_ptr(logits), rows, vocab, _ptr(fparams), _ptr(iparams), _ptr(out),
                                 self._err(), self._stream())
        self._check(rc, "sample")
        return out

    # -- a residual stream in 32-bit, mixers with state, attention over a latent, routed experts ------------------
    def rmsnorm_stream(self, h: torch.Tensor, weight: torch.Tensor, eps: float, delta: Optional[torch.Tensor] = None,
                       rows: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """RMS norm of a 32-bit stream: ``h += delta`` in 32-bit (stored back unless ``rows`` selects), then
        ``h / sqrt(mean(h^2) + eps) * weight`` rounded to ``out_dtype``.  ``weight``: fp32, one number or one a column."""
        width = h.shape[-1]
        assert h.dtype == torch.float32 and h.is_contiguous() and weight.dtype == torch.float32
        assert delta is None or (delta.is_contiguous() and delta.shape == h.shape)
        n_out = h.numel() // width if rows is None else rows.shape[0]
        out = torch.empty((n_out, width), dtype=out_dtype, device=h.device)
        rc = self.lib.pih_rmsnorm_stream(_DT[delta.dtype] if delta is not None else 0, _DT[out_dtype], _ptr(h), _ptr(delta),
                                         _ptr(weight), weight.numel(), _ptr(out), _ptr(rows), n_out, width, c_float(eps),
                                         self._stream())
        self._check(rc, "rmsnorm_stream")
        return out

    def linear_batched(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                       rotate: Optional[dict] = None, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``out[t, b] = x[t, b] . w[b]^T``: x ``[T, B, K]`` (a view whose rows may be strided), w ``[B, N, K]``;
        32-bit accumulation in ascending k; out ``[T, B, N]`` contiguous.

        ``rotate`` (the arguments of ``rotate_heads``: offset, frequencies, interleaved, positions): part of every
        ``x[t, b]`` is rotated first; ``gate`` ``[T, B N]`` (a view): the output times its sigmoid, column by column.
        Few rows in bf16 do both inside the product's kernel; otherwise ``rotate_heads`` runs before the product and
        ``gate_mul`` behind it (the same values: each step rounds where the separate kernel would)."""
        T, B, K = x.shape
        N = w.shape[1]
        out_dtype = out_dtype or x.dtype
        assert w.shape == (B, N, K) and w.is_contiguous() and x.dtype == w.dtype and x.stride(2) == 1
        fused = (x.dtype == torch.bfloat16 and T <= self.skinny_max_rows and K % 8 == 0 and K <= 12288
                 and T * B <= 65535 * 16 and (gate is None or (out_dtype == torch.bfloat16 and gate.dtype == torch.bfloat16)))
        if (rotate is not None or gate is not None) and not fused:
            if rotate is not None:
                x = self.rotate_heads(x, **rotate)
            out = self.linear_batched(x, w, out_dtype)
            if gate is not None:
                out = self.gate_mul(out.view(T, B * N), gate, "sigmoid").view(T, B, N)
            return out
        if x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 and T >= self.batched_library_min_rows:
            # many rows in bf16: the library's batched product (32-bit accumulation), as the single products of many rows
            return torch.bmm(x.transpose(0, 1), w.transpose(1, 2)).transpose(0, 1).contiguous()
        out = torch.empty(T, B, N, dtype=out_dtype, device=x.device)
        if x.dtype == torch.bfloat16 and T <= self.skinny_max_rows and K % 8 == 0:
            # few rows in bf16: a warp an output column, the small matrices' rows streamed once
            freq = rotate["frequencies"] if rotate is not None else None
            rc = self.lib.pih_batched_gemv(_DT[out_dtype], _ptr(x), c_ll(x.stride(0)), c_ll(x.stride(1)), _ptr(w), _ptr(out),
                                           T, B, N, K, _ptr(freq), _ptr(rotate["positions"] if rotate is not None else None),
                                           rotate["offset"] if rotate is not None else 0,
                                           2 * freq.shape[0] if freq is not None else 0,
                                           1 if (rotate is not None and rotate["interleaved"]) else 0, _ptr(gate),
                                           c_ll(gate.stride(0) if gate is not None else 0), self._stream())
            if rc != -2:
                self._check(rc, "batched_gemv")
                return out
            assert rotate is None and gate is None, "the few-rows batched product refused a shape it was asked to fuse"
        rc = self.lib.pih_gemm_simt_batched(_DT[x.dtype], _DT[out_dtype], _ptr(x), _ptr(w), _ptr(out), T, N, K,
                                            c_ll(x.stride(0)), c_ll(K), c_ll(B * N), B, c_ll(x.stride(1)), c_ll(N * K),
                                            c_ll(N), self._stream())
        self._check(rc, "gemm_simt_batched")
        return out

    latent_mma = True                      # bf16 attention over a latent of rank 64 ... 512: the tensor-core kernel ...
    latent_mma_min_rows = 0                # ... for steps of more rows than this
    latent_mma_rows_above = 64             # ... with blocks of 4 rows of a request from this many rows on
    latent_split = True                    # bf16 attention over a latent: keys cut into parts (False: the in-order kernel)
    batched_library_min_rows = 128         # bf16 batched products of at least this many rows are the library's

    def causal_conv(self, x: torch.Tensor, w: torch.Tensor, *, step, state: torch.Tensor, state_offset: int,
                    in_bias: Optional[torch.Tensor] = None, out_bias: Optional[torch.Tensor] = None,
                    activation: Optional[str] = None) -> torch.Tensor:
        """Short causal convolution per channel over each request's rows: x ``[T, C]`` (a view), w ``[C, taps]`` with
        the last tap on the current row; ``in_bias`` is added to x first, ``out_bias`` to the sum; ``activation``
        None or "silu".  The last ``taps - 1`` inputs of a request live in ``state[slot, state_offset:]`` as
        ``[taps - 1, C]`` (fp32), are read as the rows before the step's and are replaced by the step's last ones."""
        T, C = x.shape
        taps = w.shape[1]
        assert x.stride(1) == 1 and w.is_contiguous() and w.dtype == x.dtype and state.dtype == torch.float32
        out = torch.empty(T, C, dtype=x.dtype, device=x.device)
        rc = self.lib.pih_causal_conv(_DT[x.dtype], _ptr(x), c_ll(x.stride(0)), _ptr(w), _ptr(in_bias), _ptr(out_bias),
                                      _ptr(out), c_ll(C), C, taps, {None: 0, "silu": 1}[activation], _ptr(state),
                                      c_ll(state.stride(0)), c_ll(state_offset), _ptr(step.cu_q), _ptr(step.state_slots),
                                      T, step.num_requests, self._stream())
        self._check(rc, "causal_conv")
        self.launches += 1 if taps > 1 else 0                  # (the history's kernel)
        return out

    def gated_delta_rule(self, qkv: torch.Tensor, ba: torch.Tensor, *, decay_log, decay_bias, state: torch.Tensor, step,
                         heads: int, kv_heads: int, key_dim: int, value_dim: int, unit_eps: float,
                         q_scale: float) -> torch.Tensor:
        """The gated delta rule over the step's rows, request by request from each one's state slot
        (``state[slot, :heads * key_dim * value_dim]`` is S).  qkv ``[T, 2 kv_heads key_dim + heads value_dim]``:
        q heads, k heads, v heads after convolution and activation; ba ``[T, 2 heads]`` (a view): write-strength
        logits, decay logits.  Returns the read-outs, fp32 ``[T, heads, value_dim]``."""
        T = qkv.shape[0]
        assert qkv.stride(1) == 1 and ba.stride(1) == 1 and ba.dtype == qkv.dtype
        scratch = torch.empty(T * (2 * kv_heads * key_dim + 2 * heads), dtype=torch.float32, device=qkv.device)
        out = torch.empty(T, heads, value_dim, dtype=torch.float32, device=qkv.device)
        rc = self.lib.pih_gated_delta_rule(_DT[qkv.dtype], _ptr(qkv), c_ll(qkv.stride(0)), _ptr(ba), c_ll(ba.stride(0)),
                                           _ptr(decay_log), _ptr(decay_bias), _ptr(scratch), _ptr(out), _ptr(state),
                                           c_ll(state.stride(0)), _ptr(step.cu_q), _ptr(step.state_slots), T,
                                           step.num_requests, heads, kv_heads, key_dim, value_dim, c_float(unit_eps),
                                           c_float(q_scale), self._stream())
        self._check(rc, "gated_delta_rule")
        self.launches += 1                                     # two kernels
        return out

    def gated_rmsnorm(self, o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
        """``o / sqrt(mean(o^2) + eps) * weight * silu(gate)`` per (row, head): o fp32 ``[T, heads, vdim]``, gate
        ``[T, heads * vdim]`` (a view), weight fp32 ``[vdim]``; returns ``[T, heads * vdim]`` in the gate's dtype."""
        T, heads, vdim = o.shape
        assert o.is_contiguous() and gate.stride(1) == 1
        out = torch.empty(T, heads * vdim, dtype=gate.dtype, device=o.device)
        rc = self.lib.pih_gated_rmsnorm(_DT[gate.dtype], _ptr(o), _ptr(gate), c_ll(gate.stride(0)), _ptr(weight), _ptr(out),
                                        T, heads, vdim, c_float(eps), self._stream())
        self._check(rc, "gated_rmsnorm")
        return out

    def rglru_scan(self, u: torch.Tensor, gates: torch.Tensor, y_pre: torch.Tensor, *, y_bias, r_bias, i_bias, lam,
                   decay_scale: float, state: torch.Tensor, step, blocks: int) -> torch.Tensor:
        """Real-gated linear recurrent unit over the step's rows from each request's state (``state[slot, :W]``):
        ``a = exp(-decay_scale * sigmoid(gr + r_bias) * softplus(lam))``,
        ``S <- a S + sqrt(1 - a^2) * sigmoid(gi + i_bias) * u``, out ``= S * gelu_tanh(y_pre + y_bias)``.
        u ``[T, W]``; gates fp32 ``[T, blocks, 2 W / blocks]`` (a block's gr, then its gi); y_pre ``[T, W]`` (a view)."""
        T, W = u.shape
        assert u.stride(1) == 1 and y_pre.stride(1) == 1 and gates.is_contiguous() and gates.dtype == torch.float32
        out = torch.empty(T, W, dtype=u.dtype, device=u.device)
        coef = torch.empty(T, W, 4, dtype=torch.float32, device=u.device)     # per (row, channel): a - 1, the input's two factors, gelu(y)
        rc = self.lib.pih_rglru_scan(_DT[u.dtype], _ptr(u), c_ll(u.stride(0)), _ptr(gates), _ptr(y_pre),
                                     c_ll(y_pre.stride(0)), _ptr(y_bias), _ptr(r_bias), _ptr(i_bias), _ptr(lam),
                                     c_float(decay_scale), _ptr(coef), _ptr(out), c_ll(W), _ptr(state), c_ll(state.stride(0)),
                                     _ptr(step.cu_q), _ptr(step.state_slots), T, step.num_requests, W, blocks,
                                     self._stream())
        self._check(rc, "rglru_scan")
        self.launches += 1                                     # two kernels
        return out

    def latent_write(self, raw: torch.Tensor, weight: torch.Tensor, eps: float, cache: torch.Tensor,
                     slot_mapping: torch.Tensor, frequencies: Optional[torch.Tensor] = None, interleaved: bool = False,
                     positions: Optional[torch.Tensor] = None, query_latent: Optional[torch.Tensor] = None,
                     query_weight: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """``rmsnorm(raw) * weight`` of every row into its slot of the paged latent cache ``[pages, page_size, rank]``.
        With ``frequencies`` (fp32 ``[rot / 2]``) the rows hold ``rot`` more numbers behind the ``rank`` normed ones:
        they are not normed but rotated by ``positions[row] * f_i`` (pairs of neighbours with ``interleaved``, else
        halves) and cached behind the latent.  The cache may be wider than ``rank + rot`` (columns of padding, which
        stay as they are: zero).  ``query_latent`` ``[T, n]`` (a view) with ``query_weight`` (fp32 ``[n]``): the same
        launch norms it too (the same ``eps``) and returns it as ``[T, n]`` contiguous."""
        T, width = raw.shape
        rot = 2 * frequencies.shape[0] if frequencies is not None else 0
        rank = width - rot
        num_pages, page_size = cache.shape[0], cache.shape[1]
        assert raw.stride(1) == 1 and cache.dtype == raw.dtype and cache.shape[2] >= width and weight.shape[0] == rank
        q_out, q_rank, ldq = None, 0, 0
        if query_latent is not None:
            q_rank, ldq = query_latent.shape[1], query_latent.stride(0)
            assert query_latent.shape[0] == T and query_latent.stride(1) == 1 and query_latent.dtype == raw.dtype
            assert query_weight.dtype == torch.float32 and query_weight.shape[0] == q_rank
            q_out = torch.empty(T, q_rank, dtype=raw.dtype, device=raw.device)
        rc = self.lib.pih_latent_write(_DT[raw.dtype], _ptr(raw), c_ll(raw.stride(0)), _ptr(weight), c_float(eps),
                                       _ptr(cache), _ptr(slot_mapping), T, rank, page_size, num_pages, cache.shape[2], rot,
                                       1 if interleaved else 0, _ptr(frequencies), _ptr(positions), _ptr(query_latent),
                                       c_ll(ldq), _ptr(query_weight), _ptr(q_out), q_rank, self._err(), self._stream())
        self._check(rc, "latent_write")
        return q_out

    def latent_attention(self, q: torch.Tensor, *, gate: Optional[torch.Tensor], sink: Optional[torch.Tensor],
                         cache: torch.Tensor, block_table: torch.Tensor, step, scale: float, window: int = 0) -> torch.Tensor:
        """Causal attention of folded queries ``q [T, heads, rank]`` over the cached latents, which serve every head
        as key and as value; ``sink`` (fp32 ``[heads]``) joins the softmax denominator; ``gate [T, heads]`` (a view of
        logits) scales the output by its sigmoid.  Returns the weighted sums of latents ``[T, heads, rank]``."""
        T, heads, rank = q.shape
        num_pages, page_size = cache.shape[0], cache.shape[1]
        assert q.is_contiguous() and (gate is None or gate.stride(1) == 1)
        out = torch.empty_like(q)
        if q.dtype == torch.bfloat16 and self.latent_mma and rank in (64, 128, 192, 256, 384, 512) and T > self.latent_mma_min_rows:
            # tensor cores: the row's heads are the rows of the MMA, a tile of latents feeds every head's scores and sums;
            # a row's keys are cut into ``splits`` parts side by side, and each of a block's 8 warps is a part of its own
            # steps of many rows (prompt portions): a block is 4 consecutive rows of a request, which share a tile
            per_block = 4 if T > self.latent_mma_rows_above else 1
            blocks = (T if per_block == 1 else -(-T // 4) + step.num_requests) * (-(-heads // 16)) * (2 if rank > 256 else 1)
            splits = max(1, min(16, (2 * 148) // max(1, blocks)))
            parts = splits * 8 // per_block
            partial = torch.empty(T * heads * parts * (rank + 2), dtype=torch.float32, device=q.device)
            rc = self.lib.pih_latent_attention_mma(
                _ptr(q), _ptr(gate), c_ll(gate.stride(0) if gate is not None else 0), _ptr(sink), _ptr(cache),
                _ptr(block_table), block_table.shape[1], _ptr(step.request_of_row), _ptr(step.positions), _ptr(step.cu_q),
                step.num_requests, _ptr(partial), _ptr(out), T, heads, rank, page_size, num_pages, c_float(scale),
                int(window), splits, per_block, self._err(), self._stream())
            if rc != -2:
                self._check(rc, "latent_attention_mma")
                self.launches += 1
                return out
        if q.dtype == torch.bfloat16 and self.latent_split and rank % 4 == 0:
            # the serving path: a row's keys are cut into parts that run side by side (as many as fill the GPU for this
            # number of rows) and a tile of latents is fetched once for 8 heads.  The 32-bit path keeps the kernel that
            # visits a row's keys in order, whose result does not depend on the step's make-up by a single bit.
            splits = self.lib.pih_latent_attention_splits(T, heads)
            partial = torch.empty(T * heads * splits * (rank + 2), dtype=torch.float32, device=q.device)
            rc = self.lib.pih_latent_attention_split(
                _DT[q.dtype], _ptr(q), _ptr(gate), c_ll(gate.stride(0) if gate is not None else 0), _ptr(sink), _ptr(cache),
                _ptr(block_table), block_table.shape[1], _ptr(step.request_of_row), _ptr(step.positions), _ptr(partial),
                _ptr(out), T, heads, rank, page_size, num_pages, c_float(scale), int(window), splits, self._err(),
                self._stream())
            if rc != -2:
                self._check(rc, "latent_attention_split")
                self.launches += 1
                return out
        rc = self.lib.pih_latent_attention_generic(
            _DT[q.dtype], _ptr(q), _ptr(gate), c_ll(gate.stride(0) if gate is not None else 0), _ptr(sink), _ptr(cache),
            _ptr(block_table), block_table.shape[1], _ptr(step.request_of_row), _ptr(step.positions), _ptr(out), T, heads,
            rank, page_size, num_pages, c_float(scale), int(window), self._err(), self._stream())
        self._check(rc, "latent_attention_generic")
        return out

    moe_few_slots = 64            # bf16 steps of at most this many (row, choice) slots stream the chosen experts' rows
    moe_library_min_slots = 65    # ... and from this many on the experts' products are the library's grouped product

    def moe_experts(self, x: torch.Tensor, logits: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                    top: int, routing: Optional[dict] = None) -> torch.Tensor:
        """Routed experts: per row the ``top`` largest of ``logits`` (fp32 ``[T, experts]``) choose, the softmax over
        the chosen weighs; ``out = sum_k weight_k * W_down_e (silu(W_gate_e x) * (W_up_e x))``.  ``w_gate_up``
        ``[experts, 2 ff, hidden]`` holds an expert's gate rows and then its up rows, ``w_down`` ``[experts, hidden, ff]``.

        Routing, grouping by expert and the weighted sum are the pack's kernels.  The experts' products: in 32-bit
        the pack's grouped FMA product (an order of additions fixed by the row); in bf16 a step of few rows streams
        each chosen expert's rows once (a warp a column), and a step of many rows runs the library's grouped product
        (``torch._grouped_mm``: tensor cores, the groups' boundaries read on the device) where the pack's dense
        products of many rows are the library's too.

        ``routing`` selects the other router: scores are the softmax over all ``outputs`` (the first columns of
        ``logits``, whose rows may be longer), the choice goes by score plus ``correction`` within the
        ``groups_keep`` best of ``groups`` groups, the chosen weigh with their scores (``renormalize``: divided by
        their sum), and the outputs behind the experts that have matrices are identity experts (the row itself).
        ``routing["scoring"]`` "sigmoid": a score is the sigmoid of the output's own logit.  ``routing["gated"]`` False:
        an expert is ``W_down max(W_up x, 0)^2`` and ``w_gate_up`` is ``[experts, ff, hidden]``.  ``routing["weigh"]``
        "input": an expert reads the row times its weight (rounded to the compute dtype) and the outputs are summed
        as they are."""
        T, hidden = x.shape
        gated = routing.get("gated", True) if routing is not None else True
        weigh_input = routing is not None and routing.get("weigh", "output") == "input"
        with_matrices, ff = w_gate_up.shape[0], w_gate_up.shape[1] // (2 if gated else 1)
        experts = routing["outputs"] if routing is not None else with_matrices
        identity = experts - with_matrices
        assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[0] == T and identity >= 0
        assert logits.shape[1] >= experts if routing is not None else (logits.is_contiguous() and logits.shape[1] == experts)
        assert x.stride(1) == 1 and w_gate_up.is_contiguous() and w_down.is_contiguous()
        slots = T * top
        bf16 = x.dtype == torch.bfloat16
        vec = 8 if bf16 else 4
        few = bf16 and slots <= self.moe_few_slots and hidden % vec == 0 and ff % vec == 0 and max(hidden, ff) <= 12288
        words = self.lib.pih_moe_route_words(T, experts, top)
        # (few rows: every slot is taken on its own, nothing is grouped or counted)
        ints = (torch.empty if few else torch.zeros)(int(words), dtype=torch.int32, device=x.device)
        weight_of = torch.empty(slots, dtype=torch.float32, device=x.device)
        if routing is None:
            rc = self.lib.pih_moe_route(_ptr(logits), T, experts, top, _ptr(ints), _ptr(weight_of), 0 if few else 1,
                                        self._stream())
        else:
            rc = self.lib.pih_moe_route_scored(_ptr(logits), c_ll(logits.stride(0)), _ptr(routing.get("correction")), T,
                                               experts, top, int(routing.get("groups", 1)), int(routing.get("groups_keep", 1)),
                                               1 if routing.get("renormalize") else 0,
                                               {"softmax": 0, "sigmoid": 1}[routing.get("scoring", "softmax")], _ptr(ints),
                                               _ptr(weight_of), 0 if few else 1, self._stream())
        self._check(rc, "moe_route")
        self.launches += 0 if few else 2
        out = torch.empty(T, hidden, dtype=x.dtype, device=x.device)
        if (bf16 and not few and slots >= self.moe_library_min_slots and hidden % 8 == 0 and ff % 8 == 0
                and hasattr(torch, "_grouped_mm")):
            row_of = ints[3 * slots:4 * slots]
            ends = ints[4 * slots + experts + 1:4 * slots + experts + 1 + with_matrices]   # where each expert's rows end
            # (the rows of identity experts lie behind the last of these: the grouped products leave them alone)
            if weigh_input:
                xs = torch.empty(slots, hidden, dtype=x.dtype, device=x.device)
                rc = self.lib.pih_moe_gather_scaled(_DT[x.dtype], _ptr(x), c_ll(x.stride(0)), _ptr(ints), _ptr(weight_of),
                                                    _ptr(xs), T, experts, top, hidden, self._stream())
                self._check(rc, "moe_gather_scaled")
            else:
                xs = self.gather_rows(x, row_of) if x.is_contiguous() else x.index_select(0, row_of)
            gate_up = torch._grouped_mm(xs, w_gate_up.transpose(1, 2), offs=ends)     # [slots, 2 ff] (or [slots, ff])
            act = self.silu_mul(gate_up) if gated else self.activation(gate_up, "relu2")
            y = torch._grouped_mm(act, w_down.transpose(1, 2), offs=ends)             # [slots, hidden]
            rc = self.lib.pih_moe_combine_bf16(_ptr(y), _ptr(ints), _ptr(weight_of), _ptr(out), T, top, hidden,
                                               with_matrices, _ptr(x), c_ll(x.stride(0)), 1 if weigh_input else 0,
                                               self._stream())
            self._check(rc, "moe_combine")
            return out
        act = torch.empty(slots, ff, dtype=x.dtype, device=x.device)
        y = torch.empty(slots, hidden, dtype=torch.float32, device=x.device)
        rc = self.lib.pih_moe_experts(_DT[x.dtype], _ptr(x), c_ll(x.stride(0)), _ptr(w_gate_up), _ptr(w_down), _ptr(act),
                                      _ptr(y), _ptr(out), _ptr(ints), _ptr(weight_of), T, experts, top, hidden, ff,
                                      1 if few else 0, identity, 1 if gated else 0, 1 if weigh_input else 0, self._stream())
        self._check(rc, "moe_experts")
        self.launches += 2
        return out

    # -- norms on the sub-layers' outputs, retention, differential attention, a biased feed-forward ---------------------
    def stream_cast(self, h: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        """A 32-bit stream rounded to ``dtype``."""
        assert h.dtype == torch.float32 and h.is_contiguous()
        out = torch.empty(h.shape, dtype=dtype, device=h.device)
        rc = self.lib.pih_stream_cast(_DT[dtype], _ptr(h), _ptr(out), c_ll(h.numel()), self._stream())
        self._check(rc, "stream_cast")
        return out

    def stream_norm_add(self, h: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                        bias: Optional[torch.Tensor] = None, copy_dtype: Optional[torch.dtype] = None):
        """``h += rmsnorm(y + bias) * weight`` in place on the stream ``h`` (32-bit sums; ``h`` may be a 32-bit path's
        stream or a 32-bit stream beside a 16-bit compute dtype); with ``copy_dtype`` returns the new ``h`` rounded to
        it (what the next sub-layer reads), else None."""
        rows, width = h.shape
        assert h.dtype == torch.float32 and h.is_contiguous() and y.shape == h.shape and y.stride(1) == 1
        weight = weight if weight.dtype == torch.float32 else weight.float()
        copy = torch.empty(rows, width, dtype=copy_dtype, device=h.device) if copy_dtype is not None else None
        rc = self.lib.pih_stream_norm_add(_DT[y.dtype], _DT[copy_dtype] if copy_dtype is not None else _DT[y.dtype], _ptr(h),
                                          _ptr(y), c_ll(y.stride(0)), _ptr(bias), _ptr(weight), _ptr(copy), rows, width,
                                          c_float(eps), self._stream())
        self._check(rc, "stream_norm_add")
        return copy

    def bias_xielu(self, z: torch.Tensor, bias: Optional[torch.Tensor], alpha_positive: float,
                   alpha_negative: float) -> torch.Tensor:
        """xIELU of ``z + bias``: ``alpha_positive u^2 + u / 2`` for u > 0, else ``alpha_negative (exp(u) - 1 - u) + u / 2``
        (32-bit inside, rounded once)."""
        rows, width = z.shape
        assert z.stride(1) == 1 and (bias is None or bias.dtype == torch.float32)
        out = torch.empty(rows, width, dtype=z.dtype, device=z.device)
        rc = self.lib.pih_bias_xielu(_DT[z.dtype], _ptr(z), c_ll(z.stride(0)), _ptr(bias), _ptr(out), c_ll(rows), width,
                                     c_float(alpha_positive), c_float(alpha_negative), self._stream())
        self._check(rc, "bias_xielu")
        return out

    def add_gated(self, a: torch.Tensor, b: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        """``a + sigmoid(gate[row]) * b``: a, b ``[T, width]``; gate fp32 ``[T]`` (a view of logits), or None: ``a + b``."""
        rows, width = a.shape
        assert a.is_contiguous() and b.is_contiguous() and b.shape == a.shape and (gate is None or gate.dtype == torch.float32)
        out = torch.empty_like(a)
        rc = self.lib.pih_add_gated(_DT[a.dtype], _ptr(a), _ptr(b), _ptr(gate), c_ll(gate.stride(0) if gate is not None else 0),
                                    _ptr(out), c_ll(rows), width, self._stream())
        self._check(rc, "add_gated")
        return out

    def retention(self, qk: torch.Tensor, v: torch.Tensor, *, frequencies: Optional[torch.Tensor],
                  decay_minus_one: torch.Tensor, key_scale: float, state: torch.Tensor, step, heads: int, key_dim: int,
                  value_dim: int) -> torch.Tensor:
        """Retention over the step's rows, request by request from each one's state slot (``state[slot]`` is
        ``S [heads, key_dim, value_dim]``): q and k (``qk [T, 2 heads key_dim]``, a view) are rotated by the row's
        position with ``frequencies`` (fp32 ``[rotary_dim / 2]``; None: no rotation), k then times ``key_scale``;
        ``S <- S + decay_minus_one S + k v^T``; returns the read-outs ``S^T q``, fp32 ``[T, heads, value_dim]``."""
        T = qk.shape[0]
        assert qk.stride(1) == 1 and v.stride(1) == 1 and v.dtype == qk.dtype and state.dtype == torch.float32
        scratch = torch.empty(2 * T * heads * key_dim, dtype=torch.float32, device=qk.device)
        out = torch.empty(T, heads, value_dim, dtype=torch.float32, device=qk.device)
        rot = 2 * frequencies.shape[0] if frequencies is not None else 0
        rc = self.lib.pih_retention(_DT[qk.dtype], _ptr(qk), c_ll(qk.stride(0)), _ptr(v), c_ll(v.stride(0)), _ptr(frequencies),
                                    rot, _ptr(step.positions), _ptr(decay_minus_one), c_float(key_scale), _ptr(scratch),
                                    _ptr(out), _ptr(state), c_ll(state.stride(0)), _ptr(step.cu_q), _ptr(step.state_slots),
                                    T, step.num_requests, heads, key_dim, value_dim, self._stream())
        self._check(rc, "retention")
        self.launches += 1                                     # two kernels
        return out

    def diff_qk_prepare(self, qkv: torch.Tensor, *, q_norm, k_norm, eps: float, frequencies, positions, slot_mapping,
                        cache: torch.Tensor, write_kv: bool, heads: int, kv_heads: int, key_dim: int, value_dim: int) -> None:
        """Per-map RMS norm (fp32 weights ``[key_dim]`` or None) and rotation of the q and k maps of the rows
        ``[q: heads x 2 x key_dim | k: kv_heads x 2 x key_dim | v: kv_heads x value_dim]``: q is changed in place, and
        with ``write_kv`` k and v go to the rows' slots of ``cache [pages, page_size, kv_heads (2 key_dim + value_dim)]``
        (without it the rows hold q alone)."""
        rows = qkv.shape[0]
        num_pages, page_size, width = cache.shape
        assert qkv.stride(1) == 1 and cache.dtype == qkv.dtype and width == kv_heads * (2 * key_dim + value_dim)
        rot = 2 * frequencies.shape[0] if frequencies is not None else 0
        rc = self.lib.pih_diff_qk_prepare(_DT[qkv.dtype], _ptr(qkv), c_ll(qkv.stride(0)), _ptr(q_norm), _ptr(k_norm),
                                          c_float(eps), _ptr(frequencies), rot, _ptr(positions), _ptr(slot_mapping),
                                          _ptr(cache), page_size, num_pages, rows, heads, kv_heads, key_dim, value_dim,
                                          1 if write_kv else 0, self._err(), self._stream())
        self._check(rc, "diff_qk_prepare")

    def diff_attention(self, qkv: torch.Tensor, *, cache: torch.Tensor, block_table: torch.Tensor, step, scale: float,
                       lam: float, out_scale: float, norm_eps: float, window: int, heads: int, kv_heads: int, key_dim: int,
                       value_dim: int) -> torch.Tensor:
        """Differential attention of the step's rows (their q maps, prepared, in the first columns of ``qkv``) over the
        cache: per head ``softmax_1 v - lam * softmax_2 v``, divided by its root mean square (``norm_eps``) and times
        ``out_scale``.  Returns ``[T, heads * value_dim]`` in the compute dtype.

        32-bit: a warp a (row, head) over the row's keys in a fixed order (the result does not depend on the step's
        make-up).  bf16: requests of more than 16 rows on the tensor-core kernel when it has an instance for the
        sizes, the other rows on the warp kernel with their keys cut into parts that run side by side."""
        rows = qkv.shape[0]
        num_pages, page_size = cache.shape[0], cache.shape[1]
        out = torch.empty(rows, heads * value_dim, dtype=qkv.dtype, device=qkv.device)
        tile, small, splits, partial = 0, 1, 1, None
        if qkv.dtype == torch.bfloat16 and self.diff_attention_fast:
            plans = getattr(step, "attention_plans", None)
            plan = plans[1] if plans is not None and 1 in plans else None
            if plan is None:
                plan = self.attention_plan(step.host_cu_q, step.host_q_start, 1)
                if plans is not None:
                    plans[1] = plan
            if self.lib.pih_diff_attention_tile_takes(key_dim, value_dim) and qkv.stride(0) % 8 == 0 and cache.shape[2] % 8 == 0:
                tile, small = (1 if plan[0] > 0 else 0), (1 if plan[1] > 0 else 0)
            if small:
                # the rows of small requests: as many parts as bring the warps of the GPU to work
                # (and no more than leave a part 128 keys of the longest context that the step's tables can hold)
                splits = max(1, min(32, (148 * 16) // max(1, rows * heads), max(1, plan[2] // 128)))
                if splits > 1:
                    partial = torch.empty(rows * heads * splits * (4 + 2 * value_dim), dtype=torch.float32, device=qkv.device)
        rc = self.lib.pih_diff_attention(
            _DT[qkv.dtype], _ptr(qkv), c_ll(qkv.stride(0)), _ptr(out), _ptr(cache), _ptr(block_table), block_table.shape[1],
            _ptr(step.request_of_row), _ptr(step.positions), _ptr(step.cu_q), _ptr(getattr(step, "q_start", None)), rows,
            step.num_requests, heads, kv_heads, key_dim, value_dim, page_size, num_pages, c_float(scale), c_float(lam),
            c_float(out_scale), c_float(norm_eps), int(window), tile, small, splits, _ptr(partial), self._err(),
            self._stream())
        self._check(rc, "diff_attention")
        self.launches += tile + (1 if splits > 1 else 0) + small - 1
        return out

    diff_attention_fast = True             # False: bf16 steps use the in-order warp kernel too

    # -- several residual streams -------------------------------------------------------------------------------------
    def embed_positions(self, table: torch.Tensor, places: Optional[torch.Tensor], ids: torch.Tensor,
                        positions: torch.Tensor, streams: int = 1, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """``[rows, streams, width]``: ``table[ids] + places[positions]`` (summed in 32-bit; ``places`` None: the
        table's rows alone), the same in every stream."""
        rows, (vocab, width) = ids.shape[0], table.shape
        assert table.is_contiguous() and (places is None or (places.is_contiguous() and places.dtype == table.dtype
                                                             and places.shape[1] == width))
        out = torch.empty(rows, streams, width, dtype=out_dtype, device=table.device)
        rc = self.lib.pih_embed_positions(_DT[table.dtype], _DT[out_dtype], _ptr(table), _ptr(places), _ptr(ids),
                                          _ptr(positions), _ptr(out), rows, width, streams, vocab,
                                          places.shape[0] if places is not None else 0, self._err(), self._stream())
        self._check(rc, "embed_positions")
        return out

    def hyper_stream(self, x: torch.Tensor, y: Optional[torch.Tensor], *, mix=None, spread=None, collect=None, weight=None,
                     eps: float = 0.0, rows: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None):
        """One pass over the rows of the streams ``x`` (fp32 ``[T, S, width]``, in place).  With ``y [T, width]`` (a
        sub-layer's output that is not written yet): ``x_t <- sum_s mix[s, t] x_s + spread[t] y`` for all t at once.
        With ``collect`` (fp32 ``[S]``): returns ``u = sum_t collect[t] x_t`` of the new streams as ``[T, width]`` of
        ``out_dtype``, RMS-normed with ``weight`` (fp32 ``[width]``) and ``eps`` where a weight is given.  ``rows``
        (int32): only these rows are read, and nothing is stored.  Sums and norm are 32-bit."""
        T, S, width = x.shape
        assert x.dtype == torch.float32 and x.is_contiguous() and (y is None or (y.stride(1) == 1 and y.shape == (T, width)))
        n_out = T if rows is None else rows.shape[0]
        out = None
        if collect is not None:
            out = torch.empty(n_out, width, dtype=out_dtype or torch.float32, device=x.device)
        rc = self.lib.pih_hyper_stream(_DT[y.dtype] if y is not None else 0, _DT[out.dtype] if out is not None else 0,
                                       _ptr(x), _ptr(y), c_ll(y.stride(0) if y is not None else 0), _ptr(mix), _ptr(spread),
                                       _ptr(collect), _ptr(weight), _ptr(rows), _ptr(out), n_out, S, width, c_float(eps),
                                       self._stream())
        self._check(rc, "hyper_stream")
        return out

    # -- attention over a window with a sink --------------------------------------------------------------------------
    def window_qk_prepare(self, src: torch.Tensor, *, q_norm, k_norm, eps: float, rope_table, rotary_dim: int,
                          interleaved: bool, positions, slot_mapping, cache: torch.Tensor, heads: int, kv_heads: int,
                          key_dim: int, value_dim: int, values_from_keys: bool,
                          frequencies: Optional[torch.Tensor] = None, write_kv: bool = True) -> torch.Tensor:
        """Rows ``[q: heads x key_dim | k: kv_heads x key_dim | v: kv_heads x value_dim]`` (no v columns with
        ``values_from_keys``: the values are the key columns as they come).  q and k are RMS-normed over their whole
        width (fp32 weights a column, or None) and rotated by ``rope_table`` (fp32 ``[positions, rotary_dim / 2,
        2]``, pairs of neighbours with ``interleaved``, else halves); q is returned as ``[T, heads x key_dim]``, k and v
        go to the rows' slots of ``cache [pages, page_size, kv_heads (key_dim + value_dim)]``.  ``frequencies`` (fp32
        ``[rotary_dim / 2]``) in the table's place: the angles ``position * f_i`` are formed in 32-bit in the kernel.
        ``write_kv`` False: the rows hold q alone and nothing goes to the cache."""
        rows = src.shape[0]
        num_pages, page_size, width = cache.shape
        assert src.stride(1) == 1 and cache.dtype == src.dtype and width == kv_heads * (key_dim + value_dim)
        assert src.shape[1] >= heads * key_dim + (0 if not write_kv else
                                                   kv_heads * key_dim + (0 if values_from_keys else kv_heads * value_dim))
        assert rope_table is None or frequencies is None
        q = torch.empty(rows, heads * key_dim, dtype=src.dtype, device=src.device)
        rot = rotary_dim if (rope_table is not None or frequencies is not None) else 0
        assert frequencies is None or 2 * frequencies.shape[0] == rot
        rc = self.lib.pih_window_qk_prepare(_DT[src.dtype], _ptr(src), c_ll(src.stride(0)), _ptr(q), _ptr(q_norm),
                                            _ptr(k_norm), c_float(eps), _ptr(rope_table), _ptr(frequencies), rot,
                                            1 if interleaved else 0,
                                            rope_table.shape[0] if rope_table is not None else 0, _ptr(positions),
                                            _ptr(slot_mapping), _ptr(cache), page_size, num_pages, rows, heads, kv_heads,
                                            key_dim, value_dim, 1 if values_from_keys else 0, 1 if write_kv else 0,
                                            self._err(), self._stream())
        self._check(rc, "window_qk_prepare")
        return q

    def window_attention(self, q: torch.Tensor, *, cache: torch.Tensor, block_table: torch.Tensor, step, scale: float,
                         window: int, keep_first: int, softcap: float, bias: Optional[torch.Tensor],
                         sink: Optional[torch.Tensor], gate: Optional[torch.Tensor], heads: int, kv_heads: int,
                         key_dim: int, value_dim: int) -> torch.Tensor:
        """Attention of the step's rows (q prepared, ``[T, heads x key_dim]``) over the keys of their window and the
        kept first keys; ``bias`` fp32 ``[heads, distances]`` by distance (the last column for every larger one),
        ``softcap`` 0: none, ``sink`` fp32 ``[heads]`` or None, ``gate`` ``[T, >= heads]`` (a view: column h is head
        h's logit) or None.  Returns ``[T, heads x value_dim]``.

        32-bit: a warp a (row, head) over the row's keys in a fixed order (the result does not depend on the step's
        make-up).  bf16: requests of more than 16 rows on the tensor-core kernel when it has an instance for the
        sizes, the other rows on the warp kernel with their keys cut into parts that run side by side."""
        rows = q.shape[0]
        num_pages, page_size = cache.shape[0], cache.shape[1]
        assert q.is_contiguous() and cache.dtype == q.dtype and (gate is None or (gate.dtype == q.dtype and gate.stride(1) == 1))
        out = torch.empty(rows, heads * value_dim, dtype=q.dtype, device=q.device)
        tile, small, splits, partial = 0, 1, 1, None
        if q.dtype == torch.bfloat16 and self.window_attention_fast:
            plans = getattr(step, "attention_plans", None)
            plan = plans[1] if plans is not None and 1 in plans else None
            if plan is None:
                plan = self.attention_plan(step.host_cu_q, step.host_q_start, 1)
                if plans is not None:
                    plans[1] = plan
            if self.lib.pih_window_attention_tile_takes(key_dim, value_dim) and cache.shape[2] % 8 == 0:
                tile, small = (1 if plan[0] > 0 else 0), (1 if plan[1] > 0 else 0)
            if small:
                # a row reads at most its window and the kept keys: as many parts as bring the GPU's warps to work
                # (32 a multiprocessor: a warp waits on its loads most of the time), and no more than leave a part
                # 64 keys
                reach = plan[2] if window <= 0 else min(plan[2], window + keep_first + 32)
                splits = max(1, min(32, (148 * 32) // max(1, rows * heads), max(1, reach // 64)))
                if splits > 1:
                    per_lane = 2 if value_dim <= 64 else (4 if value_dim <= 128 else (8 if value_dim <= 256 else 16))
                    partial = torch.empty(rows * heads * splits * (2 + 32 * per_lane), dtype=torch.float32, device=q.device)
        distances = bias.shape[1] if bias is not None else 0
        rc = self.lib.pih_window_attention(
            _DT[q.dtype], _ptr(q), _ptr(out), _ptr(cache), _ptr(block_table), block_table.shape[1],
            _ptr(step.request_of_row), _ptr(step.positions), _ptr(step.cu_q), _ptr(getattr(step, "q_start", None)), rows,
            step.num_requests, heads, kv_heads, key_dim, value_dim, page_size, num_pages, c_float(scale),
            c_float(softcap or 0.0), _ptr(bias), distances, int(window), int(keep_first), _ptr(sink), _ptr(gate),
            c_ll(gate.stride(0) if gate is not None else 0), tile, small, splits, _ptr(partial), self._err(), self._stream())
        self._check(rc, "window_attention")
        self.launches += tile + (1 if splits > 1 else 0) + small - 1
        return out

    window_attention_fast = True           # False: bf16 steps use the in-order warp kernel too

    # -- a bigram embedding, rotations by computed angles, gates a column, two-matrix experts -----------------------------
    def embed_bigram(self, table: torch.Tensor, bigram: torch.Tensor, step, *, state: torch.Tensor, mul_prev: int,
                     mul_cur: int, buckets: int, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``table[token] + bigram[(previous * mul_prev + token * mul_cur) mod buckets]`` for the step's rows, summed in
        32-bit; a sequence's first token takes ``bigram[buckets]``.  The token before a request's first row of the
        step comes from ``state[slot]`` (int32 ``[slots, 1]``), where the kernel leaves the step's last token."""
        rows, (vocab, width) = step.token_ids.shape[0], table.shape
        out_dtype = out_dtype or table.dtype
        assert table.is_contiguous() and bigram.is_contiguous() and bigram.shape == (buckets + 1, width)
        assert bigram.dtype == table.dtype and state.dtype == torch.int32
        out = torch.empty(rows, width, dtype=out_dtype, device=table.device)
        rc = self.lib.pih_embed_bigram(_DT[table.dtype], _DT[out_dtype], _ptr(table), _ptr(bigram), _ptr(step.token_ids),
                                       _ptr(step.positions), _ptr(step.request_of_row), _ptr(step.cu_q),
                                       _ptr(step.state_slots), _ptr(state), c_ll(state.stride(0)), state.shape[0], _ptr(out),
                                       rows, width, vocab, c_ll(buckets), c_ll(mul_prev), c_ll(mul_cur), self._err(),
                                       self._stream())
        self._check(rc, "embed_bigram")
        return out

    def rmsnorm_rows(self, x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
        """``x / sqrt(mean(x^2) + eps) * weight`` over the columns of ``x [T, n]`` (a view whose rows may be strided),
        ``weight`` fp32 ``[n]``; returns ``[T, n]`` contiguous in the dtype of ``x``."""
        T, n = x.shape
        assert x.stride(1) == 1 and weight.dtype == torch.float32 and weight.shape[0] == n
        out = torch.empty(T, n, dtype=x.dtype, device=x.device)
        rc = self.lib.pih_rmsnorm_rows(_DT[x.dtype], _ptr(x), c_ll(x.stride(0)), _ptr(weight), _ptr(out), T, n, c_float(eps),
                                       self._stream())
        self._check(rc, "rmsnorm_rows")
        return out

    def rotate_heads(self, x: torch.Tensor, *, offset: int, frequencies: torch.Tensor, interleaved: bool,
                     positions: torch.Tensor) -> torch.Tensor:
        """``x [T, heads, width]`` (a view whose rows may be strided) with the columns ``offset .. offset + rot`` of
        every head rotated by ``positions[row] * f_i`` (32-bit angles; ``rot = 2 len(frequencies)``; pairs of neighbours
        with ``interleaved``, else halves); returns ``[T, heads, width]`` contiguous."""
        T, heads, width = x.shape
        assert x.stride(2) == 1 and x.stride(1) == width and frequencies.dtype == torch.float32
        out = torch.empty(T, heads, width, dtype=x.dtype, device=x.device)
        rc = self.lib.pih_rotate_heads(_DT[x.dtype], _ptr(x), c_ll(x.stride(0)), _ptr(out), _ptr(frequencies), _ptr(positions),
                                       T, heads, width, offset, 2 * frequencies.shape[0], 1 if interleaved else 0,
                                       self._stream())
        self._check(rc, "rotate_heads")
        return out

    def gate_mul(self, a: torch.Tensor, gate: torch.Tensor, kind: str = "sigmoid") -> torch.Tensor:
        """``a * sigmoid(gate)`` (``kind`` "silu": ``a * silu(gate)``), column by column: a ``[T, n]`` contiguous, gate
        ``[T, n]`` (a view whose rows may be strided); 32-bit inside, rounded once."""
        T, n = a.shape
        assert a.is_contiguous() and gate.shape == a.shape and gate.stride(1) == 1 and gate.dtype == a.dtype
        out = torch.empty_like(a)
        rc = self.lib.pih_gate_mul(_DT[a.dtype], _ptr(a), _ptr(gate), c_ll(gate.stride(0)), _ptr(out), c_ll(T), n,
                                   {"sigmoid": 1, "silu": 2}[kind], self._stream())
        self._check(rc, "gate_mul")
        return out

    def activation(self, z: torch.Tensor, kind: str) -> torch.Tensor:
        """``kind`` "relu2": the square of ``max(z, 0)``; z ``[T, n]`` (rows may be strided); 32-bit inside, rounded once."""
        T, n = z.shape
        assert z.stride(1) == 1
        out = torch.empty(T, n, dtype=z.dtype, device=z.device)
        rc = self.lib.pih_unary_act(_DT[z.dtype], _ptr(z), c_ll(z.stride(0)), _ptr(out), c_ll(T), n, {"relu2": 1}[kind],
                                    self._stream())
        self._check(rc, "unary_act")
        return out

    def scale_(self, x: torch.Tensor, scale: float) -> torch.Tensor:
        """``x *= scale`` in place; x fp32, contiguous."""
        assert x.dtype == torch.float32 and x.is_contiguous()
        rc = self.lib.pih_scale_rows(_ptr(x), c_ll(x.numel()), c_float(scale), self._stream())
        self._check(rc, "scale_rows")
        return x
