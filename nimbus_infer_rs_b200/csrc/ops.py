"""Tensor-level face of the kernel library.

Each function checks its tensors and hands raw pointers plus the current CUDA stream to one
``extern "C"`` launcher of ``libnimbus_b200.so``.  There is no other implementation in the
package: if the library cannot be built or loaded, the first call raises.

The functions go through a backend object so that a test can drive the engine's host logic
(batching, paging, slots) with a stand-in of its own; the package itself only ever
installs :class:`CudaBackend`.
"""
from __future__ import annotations

import os

import torch

ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF, ACT_SILU, ACT_RELU2, ACT_TANH, ACT_XIELU = 0, 1, 2, 3, 4, 5, 6
ACT_RELU = 7
ACT_SWISH_CLAMP = 8    # g = min(gate, L), u = clamp(up, -L, L): g * sigmoid(1.702 g) * (u + 1); gated halves only
# what a dense product's epilogue can apply
ACTIVATIONS = {"none": ACT_NONE, "gelu_tanh": ACT_GELU_TANH, "gelu_erf": ACT_GELU_ERF}
# what the experts' first product (routed experts) can apply
GATE_ACTIVATIONS = {**ACTIVATIONS, "silu": ACT_SILU, "relu2": ACT_RELU2}
# what the gate of a gated dense feed-forward can apply (`glu_rows`)
GLU_ACTIVATIONS = {**GATE_ACTIVATIONS, "relu": ACT_RELU, "swish_clamp": ACT_SWISH_CLAMP}
# combiners of a gated half that take a number (the bound of ``swish_clamp``)
PARAM_ACTIVATIONS = {"swish_clamp"}
# what a pass over fp32 rows can apply (`act_rows`): those, and activations with learned numbers
ROW_ACTIVATIONS = {"tanh": ACT_TANH, "xielu": ACT_XIELU}

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
DECODE_TARGET_CTAS = 4 * 148   # CTAs the split 32-bit decode attention aims to put on the GPU
# CTAs the tensor-core prefill attention aims to put on the GPU by cutting the keys of a tile
# into runs: one per SM.  (Two of its CTAs on an SM are bound by instruction issue, so cutting
# further only adds the merge; measured on GPT-2 124M, 2 x 1024 tokens.)
PREFILL_TARGET_CTAS = 148
FUSED_NORM_MAX_ROWS = 16       # a LayerNorm is folded into the product up to this many rows
FUSED_NORM_MAX_COLS = 16384    # ... and output columns (a long weight stream wants the leaner kernel)
SKINNY_MAX_ROWS = 64   # matrix products with at most this many rows take the weight-streaming kernel
STREAM_MAX_ROWS = 16   # ... and with at most this many the kernel that stages weights in shared memory
ROWS_MAX_ROWS = 128    # up to this many rows a product's weights are the tensor cores' 128-row operand
MOE_TC_MIN_PLACES = 1024   # from this many (token, choice) pairs on the experts' products take tcgen05 tiles


def decode_splits(base_ctas: int, pages: int, page: int, head_dim: int, sms: int, most: int) -> int:
    """Splits of a sequence's pages in the tensor-core decode attention (swept on a B200 at
    contexts of 256 and 1,024 and batches of 1 to 32).  Four pages a split: eight warps take
    two at a time, so a split is two turns of the loop and every page is asked for before the
    kernel's wait.  Fewer splits if the launch would be more than a third larger than what
    fits on the GPU at once with four pages in flight per CTA (512 to 576 CTAs of four warps
    still beat half as many splits, 768 do not), and only counts that deal the pages out
    evenly (three splits of 16 pages measured 10 % worse than two or four).  More, while the
    launch is still smaller than the GPU.  `most`: the largest count allowed (what merges
    inside a thread-block cluster, or 16)."""
    four_pages = 8 * page * (head_dim + 8) * 2
    room = max(1, min(8, (228 * 1024) // (four_pages + 1024))) * sms
    most = max(1, min(pages, most))
    s = max(1, min(most, -(-pages // 4)))
    while s > 1 and (s * base_ctas > room * 13 // 10 or pages % s):
        s -= 1
    while 2 * s <= most and 2 * s * base_ctas <= sms and pages % (2 * s) == 0:
        s *= 2
    return s


def latent_splits(ctas: int, pages: int, sms: int) -> int:
    """Into how many runs the tensor-core latent attention cuts the pages of a tile: one when
    the tiles alone fill the GPU, else as many as bring the launch to about two CTAs per SM,
    at most one per page and at most 32."""
    if ctas >= sms or pages < 2:
        return 1
    return max(1, min(pages, 32, (2 * sms) // max(1, ctas)))


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[t]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t}") from None


def _ptr(t: torch.Tensor | None) -> int:
    """The tensor's address (0 for None); the entry points declare their pointer arguments."""
    return 0 if t is None else t.data_ptr()


try:    # the current stream's handle without building a Stream object (a few hundred ns)
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:   # pragma: no cover
    _raw_stream = None


def _check(t: torch.Tensor, name: str, dtype=None, ndim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor, got device {t.device}")
    if not t.is_contiguous():
        raise KernelError(f"{name}: expected a contiguous tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name}: expected {ndim} dimensions, got {t.dim()}")


class CudaBackend:
    """Calls into the compiled library."""

    name = "cuda"

    def __init__(self):
        from . import build
        from .signatures import declare
        self.lib = build.load()
        declare(self.lib)
        self._device_index = torch.cuda.current_device()
        self.launches = 0  # kernels launched through this backend (for measurement reports)
        self._scratch = {}
        self._argmax_scratch = {}
        self._prefill_scr = {}
        self._latent_scr = {}
        # NIMBUS_B200_MMA=0 keeps the latent attention and the routed experts' products of a
        # bfloat16 run on the CUDA-core kernels (comparison runs)
        self.use_mma = os.environ.get("NIMBUS_B200_MMA", "1") != "0"
        # NIMBUS_B200_NO_TCGEN05=1 keeps large bf16 products on the CUDA-core kernel (debugging)
        self.use_tcgen05 = os.environ.get("NIMBUS_B200_NO_TCGEN05", "") in ("", "0")
        # NIMBUS_B200_STREAM=0 keeps a decode step's products on the kernel that streams weights
        # through registers (comparison runs)
        self.use_stream = os.environ.get("NIMBUS_B200_STREAM", "1") != "0"
        # NIMBUS_B200_ROWS=0/1/2: products of up to 128 rows on the kernel that cuts K among the
        # CTAs of a cluster: never / where it is the faster one (a long K over few columns) /
        # wherever it applies
        self.use_rows = int(os.environ.get("NIMBUS_B200_ROWS", "1") or 1)
        # NIMBUS_B200_DECODE_CLUSTERS=0: the splits of the bfloat16 decode attention merge through
        # scratch memory and a counter instead of a thread-block cluster's shared memory
        self._cluster_limit = int(self.lib.nb_attention_decode_cluster_limit())
        self._sms = torch.cuda.get_device_properties(self._device_index).multi_processor_count
        self.set_decode_clusters(int(os.environ.get("NIMBUS_B200_DECODE_CLUSTERS", "1") or 1))
        # NIMBUS_B200_OVERLAP=0/1: let a kernel's set-up and first weight fetch overlap the tail
        # of the kernel before it (programmatic dependent launch; on by default)
        self.set_overlap(os.environ.get("NIMBUS_B200_OVERLAP", "1") != "0")
        # NIMBUS_B200_PAIRS=0/1/2: large products on pairs of CTAs: never / where the cost
        # model prefers them (products of three waves of tiles and more) / wherever possible
        self.set_pairs(int(os.environ.get("NIMBUS_B200_PAIRS", "1") or 1))

    def set_pairs(self, mode) -> None:
        """Large products on pairs of CTAs sharing 256-row tiles (`cta_group::2`): 0/False off,
        1/True where the cost model prefers them, 2 wherever a paired kernel exists."""
        self.pairs = int(mode)
        self.lib.nb_gemm_tcgen05_use_pairs(self.pairs)

    def set_decode_clusters(self, on) -> None:
        """Whether 2 to 8 splits of the bfloat16 decode attention merge inside a thread-block
        cluster (the default) or through scratch memory like any other number of them."""
        self.decode_clusters = 1 if on else 0
        self.lib.nb_attention_decode_cluster_merge(self.decode_clusters)

    def set_overlap(self, on: bool) -> None:
        self.lib.nb_set_overlap((1 if on else 0))
        self.overlap = bool(on)

    # -- plumbing ---------------------------------------------------------------------
    def _stream(self) -> int:
        if _raw_stream is not None:
            return _raw_stream(self._device_index)
        return torch.cuda.current_stream().cuda_stream

    def _call(self, fn_name: str, *args) -> None:
        rc = getattr(self.lib, fn_name)(*args)
        self.launches += 1
        if rc != 0:
            msg = self.lib.nb_last_error().decode("utf-8", "replace")
            raise KernelError(f"{fn_name} failed ({rc}): {msg}")

    # -- row-wise ---------------------------------------------------------------------
    def embed_pos(self, tokens, pos, wte, wpe, out, scale=1.0):
        _check(tokens, "tokens", torch.int32, 1)
        _check(pos, "pos", torch.int32, 1)
        _check(wte, "wte", None, 2)
        _check(out, "out", torch.float32, 2)
        if wpe is not None:
            _check(wpe, "wpe", wte.dtype, 2)
        n, d = out.shape
        if tokens.numel() < n or pos.numel() < n or wte.shape[1] != d:
            raise KernelError("embed_pos: shapes do not agree")
        self._call("nb_embed_pos", _ptr(tokens), _ptr(pos), _ptr(wte), _ptr(wpe),
                   dtype_code(wte.dtype), _ptr(out), n, d, float(scale), self._stream())

    def embed_hashed(self, layout, wte, pair, last, out, scale, mul_prev, mul_cur, n_buckets):
        """``out[r] = scale * wte[token] + pair[(prev * mul_prev + token * mul_cur) % n_buckets]``
        (row ``n_buckets`` of ``pair`` for a sequence's first token); ``prev`` is the row before
        in the step or, at the start of a continued sequence, ``last[slot, 0]`` (fp32 state),
        which then takes the token of the sequence's last row in this step."""
        _check(wte, "wte", None, 2)
        _check(pair, "pair", wte.dtype, 2)
        _check(last, "last", torch.float32, 2)
        _check(out, "out", torch.float32, 2)
        n, d = out.shape
        if layout.tokens.numel() < n or wte.shape[1] != d or pair.shape != (n_buckets + 1, d):
            raise KernelError("embed_hashed: shapes do not agree")
        self._call("nb_embed_hashed", _ptr(layout.tokens), _ptr(layout.row_pos), _ptr(layout.row_slot),
                   _ptr(layout.cu_rows), layout.n_seqs, _ptr(wte), _ptr(pair), dtype_code(wte.dtype),
                   _ptr(last), last.stride(0), _ptr(out), n, d, float(scale), int(mul_prev),
                   int(mul_cur), int(n_buckets), self._stream())

    def layernorm(self, x, gamma, beta, eps, out, rows=None):
        _check(x, "x", torch.float32, 2)
        _check(gamma, "gamma", torch.float32, 1)
        if beta is not None:
            _check(beta, "beta", torch.float32, 1)
        _check(out, "out", None, 2)
        if rows is not None:
            _check(rows, "rows", torch.int32, 1)
        n, d = out.shape
        if x.shape[1] != d or gamma.numel() != d or (rows is None and x.shape[0] < n):
            raise KernelError("layernorm: shapes do not agree")
        self._call("nb_layernorm", _ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out),
                   dtype_code(out.dtype), n, d, eps, self._stream())

    def rmsnorm(self, x, gamma, eps, out, rows=None, x_col=0):
        """out[r] = rms-norm of columns ``x_col .. x_col + d`` of row ``rows[r]`` (or ``r``) of the
        fp32 matrix ``x``, times ``gamma`` (or 1 if ``None``); statistics in fp32."""
        _check(x, "x", torch.float32, 2)
        _check(out, "out", None, 2)
        if gamma is not None:
            _check(gamma, "gamma", torch.float32, 1)
        if rows is not None:
            _check(rows, "rows", torch.int32, 1)
        n, d = out.shape
        if x.shape[1] < x_col + d or (gamma is not None and gamma.numel() != d) or (
                rows is None and x.shape[0] < n):
            raise KernelError("rmsnorm: shapes do not agree")
        self._call("nb_rmsnorm", _ptr(x), x.shape[1], x_col, _ptr(rows), _ptr(gamma), _ptr(out),
                   dtype_code(out.dtype), n, d, eps, self._stream())

    def ln_add(self, y, gamma, eps, residual, next_gamma, next_eps, out_next, out_cast):
        """:meth:`rms_add` with both norms centred: ``residual += (y - mean) / sqrt(var + eps) *
        gamma`` (a layer norm with a weight and no shift), ``out_next`` likewise."""
        self._norm_add("nb_ln_add", y, gamma, eps, residual, next_gamma, next_eps, out_next, out_cast)

    def rms_add(self, y, gamma, eps, residual, next_gamma, next_eps, out_next, out_cast):
        """``residual += y / sqrt(mean(y^2) + eps) * gamma`` per row (fp32), and in the same pass,
        where asked for, ``out_next = rms-norm(residual) * next_gamma`` and ``out_cast =
        residual`` in the activation type."""
        self._norm_add("nb_rms_add", y, gamma, eps, residual, next_gamma, next_eps, out_next, out_cast)

    def _norm_add(self, fn, y, gamma, eps, residual, next_gamma, next_eps, out_next, out_cast):
        _check(y, "y", torch.float32, 2)
        _check(residual, "residual", torch.float32, 2)
        _check(gamma, "gamma", torch.float32, 1)
        n, d = residual.shape
        if y.shape != residual.shape or gamma.numel() != d:
            raise KernelError("rms_add: shapes do not agree")
        code = 0
        for t, nm in ((out_next, "out_next"), (out_cast, "out_cast")):
            if t is not None:
                _check(t, nm, None, 2)
                if t.shape != residual.shape:
                    raise KernelError(f"rms_add: {nm} shape does not match")
                code = dtype_code(t.dtype)
        if out_next is not None and out_cast is not None and out_next.dtype != out_cast.dtype:
            raise KernelError("rms_add: the two outputs differ in type")
        if out_next is not None:
            _check(next_gamma, "next_gamma", torch.float32, 1)
        self._call(fn, _ptr(y), _ptr(gamma), float(eps), _ptr(residual),
                   _ptr(next_gamma if out_next is not None else None), float(next_eps),
                   _ptr(out_next), _ptr(out_cast), code, n, d, self._stream())

    def act_rows(self, x, x_col, act, params, out):
        """``out[r, i] = act(x[r, x_col + i])`` for fp32 rows ``x``: ``ACT_TANH``, or ``ACT_XIELU``
        with its two learned numbers in ``params`` (fp32 ``[2]``), or an epilogue activation."""
        _check(x, "x", torch.float32, 2)
        _check(out, "out", None, 2)
        if params is not None:
            _check(params, "params", torch.float32, 1)
        n, d = out.shape
        if x.shape[0] < n or x.shape[1] < x_col + d:
            raise KernelError("act_rows: shapes do not agree")
        self._call("nb_act_rows", _ptr(x), x.shape[1], x_col, int(act), _ptr(params), _ptr(out),
                   dtype_code(out.dtype), n, d, self._stream())

    def gather_mul(self, g, table, tokens, out):
        """``out[r] = g[r] * table[tokens[r]]`` (fp32 gate ``g``; zeros for padding rows)."""
        _check(g, "g", torch.float32, 2)
        _check(table, "table", None, 2)
        _check(tokens, "tokens", torch.int32, 1)
        _check(out, "out", None, 2)
        n, d = out.shape
        if g.shape != out.shape or table.shape[1] != d or tokens.numel() < n:
            raise KernelError("gather_mul: shapes do not agree")
        self._call("nb_gather_mul", _ptr(g), _ptr(table), dtype_code(table.dtype), _ptr(tokens),
                   _ptr(out), dtype_code(out.dtype), n, d, self._stream())

    # -- matrix products --------------------------------------------------------------
    def linear(self, x, w, bias, out, act=ACT_NONE, residual=None, norm=None):
        """out = act(norm(x) @ w.T + bias) (+ residual).  x [M,K], w [N,K], out [M,N].
        ``norm``: ``(gamma, beta, eps, act_dtype)`` asks for LayerNorm of the fp32 rows ``x``
        first; it is fused into the product where the kernel can, else run on its own."""
        _check(x, "x", None, 2)
        _check(w, "w", None, 2)
        _check(out, "out", None, 2)
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
            raise KernelError(f"linear: shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, "
                              f"out {tuple(out.shape)}")
        if bias is not None:
            _check(bias, "bias", torch.float32, 1)
            if bias.numel() != N:
                raise KernelError("linear: bias length does not match")
        if residual is not None:
            _check(residual, "residual", torch.float32, 2)
            if residual.shape != out.shape:
                raise KernelError("linear: residual shape does not match")
        tensor_core = (x.dtype == torch.bfloat16 or norm is not None and norm[3] == torch.bfloat16) \
            and w.dtype == torch.bfloat16 and K % 8 == 0 and self.use_tcgen05
        # few rows: the weight-streaming kernel; from 17 rows on the tensor-core kernel streams
        # weights faster (TMA ring), where it applies
        skinny = (M <= FUSED_NORM_MAX_ROWS or (M <= SKINNY_MAX_ROWS and not tensor_core)) \
            and (K * 32 <= 220 * 1024 if w.dtype == torch.float32 else K % 8 == 0)
        # a decode step's products (at most 16 rows, bf16 weights): weights into shared memory
        # before the kernel waits for its predecessor, so that they stream across kernel ends
        if self.use_stream and M <= STREAM_MAX_ROWS and w.dtype == torch.bfloat16 and K % 8 == 0 \
                and (norm is None or norm[3] == torch.bfloat16):
            fused = norm is not None and self.lib.nb_gemm_stream_supported(M, N, K, 1)
            if fused or self.lib.nb_gemm_stream_supported(M, N, K, 0):
                if norm is not None and not fused:
                    h = torch.empty((M, K), device=x.device, dtype=norm[3])
                    self.layernorm(x, norm[0], norm[1], norm[2], h)
                    x, norm = h, None
                gamma, beta, eps = (norm[0], norm[1], norm[2]) if norm is not None else (None, None, 0.0)
                self._call("nb_gemm_stream", _ptr(x), dtype_code(x.dtype), _ptr(gamma), _ptr(beta), eps,
                           _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), dtype_code(out.dtype), M, N,
                           K, act, self._stream())
                return
        if skinny:
            if norm is not None and (M > FUSED_NORM_MAX_ROWS or N > FUSED_NORM_MAX_COLS
                                     or w.dtype != torch.bfloat16
                                     or not self.lib.nb_gemm_skinny_norm_supported(M, N, K)):
                h = torch.empty((M, K), device=x.device, dtype=norm[3])
                self.layernorm(x, norm[0], norm[1], norm[2], h)
                x, norm = h, None
            gamma, beta, eps = (norm[0], norm[1], norm[2]) if norm is not None else (None, None, 0.0)
            self._call("nb_gemm_skinny", _ptr(x), dtype_code(x.dtype), _ptr(gamma),
                       _ptr(beta), eps, _ptr(w), dtype_code(w.dtype), _ptr(bias),
                       _ptr(residual), _ptr(out), dtype_code(out.dtype), M, N,
                       K, act, self._stream())
            return
        if norm is not None:
            h = torch.empty((M, K), device=x.device, dtype=norm[3])
            self.layernorm(x, norm[0], norm[1], norm[2], h)
            x = h
        # up to 128 rows with a long K over few columns (the MLP's second product of a decode
        # step of a larger batch or of a short prompt): weights as the 128-row operand, K cut
        # among the CTAs of a cluster
        if self.use_tcgen05 and self.use_rows and M <= ROWS_MAX_ROWS and x.dtype == torch.bfloat16 \
                and w.dtype == torch.bfloat16 and (
                    self.lib.nb_gemm_tc_rows_preferred(M, N, K) if self.use_rows == 1
                    else self.lib.nb_gemm_tc_rows_supported(M, N, K)):
            self._call("nb_gemm_tc_rows", _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                       dtype_code(out.dtype), M, N, K, act, self._stream())
            return
        if self.use_tcgen05 and self.lib.nb_gemm_tcgen05_supported(
                dtype_code(x.dtype), dtype_code(w.dtype), M, N, K):
            self._call("nb_gemm_tcgen05", _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                       dtype_code(out.dtype), M, N, K, act,
                       self._stream())
            return
        self._call("nb_gemm_simt", _ptr(x), dtype_code(x.dtype), _ptr(w),
                   dtype_code(w.dtype), _ptr(bias), _ptr(residual), _ptr(out),
                   dtype_code(out.dtype), M, N, K, act,
                   self._stream())

    # A kernel whose bounded wait on a barrier ran out says so in a word of pinned host memory
    # (one per kernel family); its results are not valid.
    _ERROR_WORDS = {0: "gemm_tcgen05", 1: "attention_prefill_tc", 2: "wait_probe", 3: "gemm_stream",
                    4: "gemm_tc_rows"}

    def raise_device_errors(self) -> None:
        """Raise if a kernel that has finished reported a timed-out wait.  Reads host memory
        only: call it where the host has already waited for the work it hands out (logits
        copied to the host, sampled tokens read back)."""
        mask = self.lib.nb_device_errors(1)
        if mask:
            names = [self._ERROR_WORDS.get(i, f"word {i}") for i in range(16) if mask >> i & 1]
            raise KernelError(f"{', '.join(names)}: a wait on a shared-memory barrier ran out of "
                              "time; results of the steps since the last check are not valid")

    def check_device_errors(self) -> None:
        """Wait for the device, then raise if a kernel reported a timed-out wait."""
        torch.cuda.synchronize(self._device_index)
        self.raise_device_errors()

    def set_wait_budget(self, cycles: int | None) -> None:
        """Clock cycles a wait on a barrier may take in the tensor-core kernels before the
        kernel gives up and reports it (``None``: the default, about two seconds)."""
        cycles = 4_000_000_000 if cycles is None else int(cycles)
        for fn in ("nb_gemm_tcgen05_set_wait_budget", "nb_attention_prefill_tc_set_wait_budget",
                   "nb_gemm_stream_set_wait_budget", "nb_gemm_tc_rows_set_wait_budget",
                   "nb_moe_gemm_tc_set_wait_budget"):
            rc = getattr(self.lib, fn)(cycles)
            if rc != 0:
                raise KernelError(f"{fn} failed ({rc}): "
                                  + self.lib.nb_last_error().decode("utf-8", "replace"))

    def wait_probe(self) -> int:
        """Run the kernels' bounded wait on a barrier that nothing completes; returns 2 if it
        gave up after the budget (the error word is then raised), 1 if it came back complete."""
        status = torch.zeros(1, dtype=torch.int32, device=f"cuda:{self._device_index}")
        self._call("nb_wait_probe", _ptr(status), self._stream())
        return int(status.item())

    # -- cache and attention ----------------------------------------------------------
    def _decode_splits(self, base_ctas: int, pages: int, kv, dtype) -> int:
        """Into how many splits a decode launch cuts each sequence's pages (`base_ctas`: rows x
        key-value heads).  The 32-bit kernel aims at a fixed number of CTAs; the tensor-core
        kernel follows `decode_splits`."""
        if dtype != torch.bfloat16:
            return max(1, min(pages, DECODE_TARGET_CTAS // base_ctas))
        return decode_splits(base_ctas, pages, kv.page, kv.head_dim, self._sms,
                             self._cluster_limit if self.decode_clusters else 16)

    def _decode_scratch(self, device, n_rows, n_heads, n_kv_heads, head_dim, n_splits):
        """Scratch of the split decode attention: partial sums per (row, head, split) and one
        counter per (row, key/value head).  Kept and grown as needed; the counters start at
        zero and every launch leaves them at zero."""
        need_acc = n_rows * n_heads * n_splits * head_dim
        need_ml = n_rows * n_heads * n_splits * 2
        need_cnt = n_rows * n_kv_heads
        s = self._scratch.get(device)
        if s is None or s[0].numel() < need_acc or s[1].numel() < need_ml or s[2].numel() < need_cnt:
            s = (torch.empty(max(need_acc, 1 << 16), dtype=torch.float32, device=device),
                 torch.empty(max(need_ml, 1 << 12), dtype=torch.float32, device=device),
                 torch.zeros(max(need_cnt, 1 << 12), dtype=torch.int32, device=device))
            self._scratch[device] = s
        return s

    def scratch_refs(self):
        """The scratch tensors kernels currently use: whoever records launches in a CUDA graph
        keeps these alive with it (growing a scratch buffer replaces the tensor)."""
        return (dict(self._scratch), dict(self._argmax_scratch), dict(self._prefill_scr),
                dict(self._latent_scr))

    def _prefill_scratch(self, device, n_tiles, max_splits, head_dim):
        """Scratch of the split prefill attention: one record per (tile, split) and one counter
        per tile; the counters start at zero and every launch leaves them at zero."""
        rec = self.lib.nb_attention_prefill_tc_record(head_dim)
        need = n_tiles * max_splits * rec
        s = self._prefill_scr.get(device)
        if s is None or s[0].numel() < need or s[1].numel() < n_tiles:
            s = (torch.empty(max(need, 1 << 20), dtype=torch.float32, device=device),
                 torch.zeros(max(n_tiles, 1 << 12), dtype=torch.int32, device=device))
            self._prefill_scr[device] = s
        return s

    def kv_append(self, src, k_col, v_col, row_slot, row_pos, kv, n_rows):
        _check(src, "src", kv.k.dtype, 2)
        self._call("nb_kv_append", _ptr(src), dtype_code(src.dtype), src.shape[1],
                   k_col, v_col, _ptr(row_slot), _ptr(row_pos), _ptr(kv.k),
                   _ptr(kv.v), _ptr(kv.block_table), kv.block_table.shape[1],
                   kv.page, kv.n_kv_heads, kv.head_dim, n_rows,
                   self._stream())

    def attention_takes(self, q_src, q_col, layout, kv, n_heads, out, scale) -> bool:
        """Whether ``attention`` has a kernel with a cap and a sink for these rows: the decode
        kernel, or the tensor-core kernel for prompts (bf16, heads of 64 or 128)."""
        if kv.v is None or q_src.dtype != kv.k.dtype:
            return False
        code = dtype_code(q_src.dtype)
        if layout.is_decode:
            return bool(self.lib.nb_attention_decode_supported(code, kv.head_dim, n_heads,
                                                               kv.n_kv_heads, kv.page)) and \
                (q_src.dtype != torch.bfloat16 or (q_src.shape[1] % 8 == 0 and q_col % 2 == 0))
        return bool(self.use_tcgen05 and scale > 0 and self.lib.nb_attention_prefill_tc_supported(
            code, kv.head_dim, n_heads, kv.n_kv_heads, kv.page, q_src.shape[1], q_col,
            dtype_code(out.dtype), out.shape[1]))

    def attention(self, q_src, q_col, layout, kv, n_heads, out, scale, window=0, append=None,
                  softcap=0.0, sink=None):
        """Causal attention of the packed rows of ``layout`` over the cache ``kv``.
        ``append=(k_col, v_col)``: the rows of ``q_src`` also hold this step's keys and values
        at those columns; they are written to the cache as well (inside the decode kernel and,
        for sequences that start at a page boundary, inside the tensor-core prefill kernel;
        else by a pass of their own before the attention kernel).  ``softcap`` > 0 replaces a
        score by ``softcap * tanh(score / softcap)``; ``sink`` (fp32 ``[n_heads]``) adds one
        term ``exp(sink_h)`` to the softmax's denominator.  With either, the decode kernel and
        the tensor-core prompt kernel are the only ones here: the caller asks
        ``attention_takes`` first."""
        capped = bool(softcap and softcap > 0) or sink is not None
        if capped and (append or not self.attention_takes(q_src, q_col, layout, kv, n_heads, out, scale)):
            raise KernelError("attention: no kernel with a cap or a sink takes this shape")
        _check(q_src, "q", kv.k.dtype, 2)
        _check(out, "out", None, 2)
        n_rows = layout.n_rows
        if out.shape[0] < n_rows or out.shape[1] != n_heads * kv.head_dim:
            raise KernelError("attention: output shape does not match")
        if layout.is_decode and self.lib.nb_attention_decode_supported(
                dtype_code(q_src.dtype), kv.head_dim, n_heads,
                kv.n_kv_heads, kv.page):
            pages = max(1, -(-layout.max_kv_len // kv.page))
            n_splits = self._decode_splits(n_rows * kv.n_kv_heads, pages, kv, q_src.dtype)
            acc, ml, counters = self._decode_scratch(q_src.device, n_rows, n_heads, kv.n_kv_heads,
                                                     kv.head_dim, n_splits)
            if capped:
                self._call("nb_attention_decode_capped", _ptr(q_src), dtype_code(q_src.dtype),
                           q_src.shape[1], q_col, _ptr(layout.row_slot), _ptr(layout.row_pos),
                           _ptr(kv.k), _ptr(kv.v), _ptr(kv.block_table), kv.block_table.shape[1],
                           kv.page, n_heads, kv.n_kv_heads, kv.head_dim, _ptr(out),
                           dtype_code(out.dtype), out.shape[1], scale, float(softcap or 0.0),
                           _ptr(sink), window, 0, 0, _ptr(None), 0, 0, n_rows, n_splits, _ptr(acc), _ptr(ml),
                           _ptr(counters), self._stream())
                return
            self._call("nb_attention_decode", _ptr(q_src), dtype_code(q_src.dtype),
                       q_src.shape[1], q_col, _ptr(layout.row_slot),
                       _ptr(layout.row_pos), _ptr(kv.k), _ptr(kv.v), _ptr(kv.block_table),
                       kv.block_table.shape[1], kv.page, n_heads,
                       kv.n_kv_heads, kv.head_dim, _ptr(out),
                       dtype_code(out.dtype), out.shape[1], scale,
                       window, n_rows, n_splits, _ptr(acc), _ptr(ml),
                       _ptr(counters), (1 if append else 0),
                       (append[0] if append else 0), (append[1] if append else 0),
                       self._stream())
            return
        if (not layout.is_decode) and self.use_tcgen05 and scale > 0 and self.lib.nb_attention_prefill_tc_supported(
                dtype_code(q_src.dtype), kv.head_dim, n_heads, kv.n_kv_heads, kv.page,
                q_src.shape[1], q_col, dtype_code(out.dtype), out.shape[1]):
            # 5th-generation tensor cores, scores in tensor memory.  When every sequence's cached
            # length is a whole number of pages (prompts from their first token, chunks cut at
            # page ends) the kernel reads the step's keys and values from the step's rows and
            # writes them to the cache itself; else they are appended first.
            fused = bool(append) and append[0] % 8 == 0 and append[1] % 8 == 0 and \
                all(p % kv.page == 0 for p in layout.seq_pos0_host)
            if append and not fused:
                self.kv_append(q_src, append[0], append[1], layout.row_slot, layout.row_pos, kv, n_rows)
            if layout.n_rows > layout.n_tokens:
                out[layout.n_tokens:layout.n_rows].zero_()      # padding rows
            # A CTA takes a 128-row tile of one head.  When there are too few of them to fill
            # the GPU, the pages a tile reads are cut into up to four runs of at least four
            # pages, one CTA each, and merged by the CTA that finishes last.
            tiles = -(-layout.max_q_len // 128)
            ctas = tiles * n_heads * layout.n_seqs
            pages = -(-layout.max_kv_len // kv.page)
            if window > 0:
                pages = min(pages, (window + 127) // kv.page + 2)
            max_splits = 1
            if 2 * ctas <= PREFILL_TARGET_CTAS and pages >= 8:
                max_splits = min(4, PREFILL_TARGET_CTAS // ctas, pages // 4)
            chunk = -(-pages // max_splits)
            part = counters = None
            if max_splits > 1:
                part, counters = self._prefill_scratch(q_src.device, ctas, max_splits, kv.head_dim)
            self._call("nb_attention_prefill_tc_capped", _ptr(q_src), dtype_code(q_src.dtype),
                       q_src.shape[1], q_col, q_src.shape[0], _ptr(layout.cu_rows),
                       _ptr(layout.seq_slot), _ptr(layout.seq_pos0), _ptr(kv.k), _ptr(kv.v),
                       kv.k.shape[0], _ptr(kv.block_table), kv.block_table.shape[1], kv.page,
                       n_heads, kv.n_kv_heads, kv.head_dim, _ptr(out), dtype_code(out.dtype),
                       out.shape[1], scale, float(softcap or 0.0), _ptr(sink), window,
                       layout.n_seqs, layout.max_q_len,
                       max_splits, chunk, _ptr(part), _ptr(counters), 1 if fused else 0,
                       append[0] if fused else 0, append[1] if fused else 0, self._stream())
            return
        if append:
            self.kv_append(q_src, append[0], append[1], layout.row_slot, layout.row_pos, kv, n_rows)
        if (not layout.is_decode) and self.lib.nb_attention_prefill_supported(
                dtype_code(q_src.dtype), kv.head_dim, n_heads,
                kv.n_kv_heads, kv.page, q_src.shape[1], q_col):
            if layout.n_rows > layout.n_tokens:
                out[layout.n_tokens:layout.n_rows].zero_()      # padding rows
            self._call("nb_attention_prefill", _ptr(q_src), dtype_code(q_src.dtype),
                       q_src.shape[1], q_col, _ptr(layout.cu_rows),
                       _ptr(layout.seq_slot), _ptr(layout.seq_pos0), _ptr(kv.k), _ptr(kv.v),
                       _ptr(kv.block_table), kv.block_table.shape[1], kv.page,
                       n_heads, kv.n_kv_heads, kv.head_dim, _ptr(out),
                       dtype_code(out.dtype), out.shape[1], scale,
                       window, layout.n_seqs, layout.max_q_len, self._stream())
            return
        if (not layout.is_decode) and q_src.dtype == torch.float32 and \
                self.lib.nb_attention_prefill_f32_supported(kv.head_dim, n_heads, kv.n_kv_heads, kv.page):
            # the 32-bit path's prompts: tiles of 64 rows, fp32 multiply-adds
            if layout.n_rows > layout.n_tokens:
                out[layout.n_tokens:layout.n_rows].zero_()      # padding rows
            self._call("nb_attention_prefill_f32", _ptr(q_src), dtype_code(q_src.dtype), q_src.shape[1],
                       q_col, _ptr(layout.cu_rows), _ptr(layout.seq_slot), _ptr(layout.seq_pos0),
                       _ptr(kv.k), _ptr(kv.v), _ptr(kv.block_table), kv.block_table.shape[1], kv.page,
                       n_heads, kv.n_kv_heads, kv.head_dim, _ptr(out), dtype_code(out.dtype),
                       out.shape[1], scale, window, layout.n_seqs, layout.max_q_len, self._stream())
            return
        self._call("nb_attention_generic", _ptr(q_src), dtype_code(q_src.dtype),
                   q_src.shape[1], q_col, _ptr(layout.row_slot), _ptr(layout.row_pos),
                   _ptr(kv.k), _ptr(kv.v), _ptr(kv.block_table), kv.block_table.shape[1],
                   kv.page, n_heads, kv.n_kv_heads, kv.head_dim,
                   _ptr(out), dtype_code(out.dtype), out.shape[1], scale,
                   window, n_rows, self._stream())

    # -- attention over a cached latent ------------------------------------------------
    def latent_append(self, src, col, gamma, eps, layout, kv):
        """The step's latents into the one-plane paged store ``kv``: columns ``col .. col +
        kv.head_dim`` of the fp32 rows ``src``, rms-normed (times ``gamma``) on the way."""
        _check(src, "src", torch.float32, 2)
        if gamma is not None:
            _check(gamma, "gamma", torch.float32, 1)
        if kv.n_kv_heads != 1 or src.shape[1] < col + kv.head_dim:
            raise KernelError("latent_append: the store must have one head of the latent's size")
        self._call("nb_latent_append", _ptr(src), src.shape[1], col, _ptr(gamma), eps,
                   _ptr(layout.row_slot), _ptr(layout.row_pos), _ptr(kv.k), dtype_code(kv.k.dtype),
                   _ptr(kv.block_table), kv.block_table.shape[1], kv.page, kv.head_dim,
                   layout.n_rows, self._stream())

    def head_linear(self, x, x_col, w, out, layout, gate=None, gate_col=0):
        """A linear map per head: ``out[r, h] = w[h] @ x[r, x_col + h*n_in : ...]`` with ``w``
        ``[n_heads, n_out, n_in]``; with ``gate`` (fp32 rows, head ``h``'s logit at column
        ``gate_col + h``) the head's result is multiplied by the logit's sigmoid."""
        _check(x, "x", None, 2)
        _check(w, "w", None, 3)
        _check(out, "out", None, 2)
        n_heads, n_out, n_in = w.shape
        n = layout.n_rows
        if x.shape[0] < n or out.shape[0] < n or x.shape[1] < x_col + n_heads * n_in \
                or out.shape[1] != n_heads * n_out:
            raise KernelError("head_linear: shapes do not agree")
        if gate is not None:
            _check(gate, "gate", torch.float32, 2)
            if gate.shape[0] < n or gate.shape[1] < gate_col + n_heads:
                raise KernelError("head_linear: gate shape does not match")
        if self.use_mma and self.lib.nb_head_linear_mma_supported(
                dtype_code(x.dtype), dtype_code(w.dtype), dtype_code(out.dtype), x.shape[1], x_col, n_in):
            self._call("nb_head_linear_mma", _ptr(x), dtype_code(x.dtype), x.shape[1], x_col, _ptr(w),
                       _ptr(out), out.shape[1], _ptr(gate), gate.shape[1] if gate is not None else 0,
                       gate_col, _ptr(layout.row_slot), n, n_heads, n_in, n_out, self._stream())
            return
        self._call("nb_head_linear", _ptr(x), dtype_code(x.dtype), x.shape[1], x_col, _ptr(w),
                   dtype_code(w.dtype), _ptr(out), dtype_code(out.dtype), out.shape[1], _ptr(gate),
                   gate.shape[1] if gate is not None else 0, gate_col, _ptr(layout.row_slot), n,
                   n_heads, n_in, n_out, self._stream())

    def attention_latent(self, q, layout, kv, n_heads, sink, out, scale, window=0):
        """Causal attention of the packed rows over the cached latents of ``kv`` (one plane: a
        token's latent is its key and its value, for every head).  ``q``: the heads' queries
        mapped into the latent's space, ``[rows, n_heads * rank]``; ``sink``: fp32 ``[n_heads]``
        logits of a key-less, value-less term of the softmax's denominator, or ``None``."""
        _check(q, "q", None, 2)
        _check(out, "out", None, 2)
        rank = kv.head_dim
        n = layout.n_rows
        if kv.n_kv_heads != 1 or q.shape[1] != n_heads * rank or out.shape[1] != n_heads * rank \
                or q.shape[0] < n or out.shape[0] < n:
            raise KernelError("attention_latent: shapes do not agree")
        if sink is not None:
            _check(sink, "sink", torch.float32, 1)
            if sink.numel() != n_heads:
                raise KernelError("attention_latent: one sink per head")
        if self.use_mma and q.dtype == out.dtype == kv.k.dtype == torch.bfloat16 \
                and self.lib.nb_attention_latent_mma_supported(rank, kv.page, n_heads):
            # tensor cores: 64 (token, head) pairs a CTA; the pages of a tile are cut into runs
            # when the launch would leave SMs idle (one-token steps, short prompts)
            ctas = -(-layout.max_q_len * n_heads // 64) * layout.n_seqs
            pages = max(1, -(-layout.max_kv_len // kv.page))
            if window > 0:
                pages = min(pages, (window + kv.page - 1) // kv.page + 2)
            n_splits = latent_splits(ctas, pages, self._sms)
            part_o = part_ml = None
            if n_splits > 1:
                need = n * n_heads * n_splits
                scr = self._latent_scr.get(q.device)
                if scr is None or scr[1].numel() < need * 2 or scr[0].numel() < need * rank:
                    scr = (torch.empty(max(need * rank, 1 << 20), dtype=torch.float32, device=q.device),
                           torch.empty(max(need * 2, 1 << 14), dtype=torch.float32, device=q.device))
                    self._latent_scr[q.device] = scr
                part_o, part_ml = scr
                self.launches += 1          # the merge
            elif layout.n_rows > layout.n_tokens:
                out[layout.n_tokens:layout.n_rows].zero_()      # padding rows
            self._call("nb_attention_latent_mma", _ptr(q), _ptr(layout.cu_rows), _ptr(layout.seq_slot),
                       _ptr(layout.seq_pos0), _ptr(layout.row_slot), _ptr(kv.k), _ptr(kv.block_table),
                       kv.block_table.shape[1], kv.page, n_heads, rank, _ptr(sink), _ptr(out), scale,
                       window, n, layout.n_seqs, layout.max_q_len, n_splits, _ptr(part_o),
                       _ptr(part_ml), self._stream())
            return
        self._call("nb_attention_latent", _ptr(q), dtype_code(q.dtype), q.shape[1], 0,
                   _ptr(layout.row_slot), _ptr(layout.row_pos), _ptr(kv.k), dtype_code(kv.k.dtype),
                   _ptr(kv.block_table), kv.block_table.shape[1], kv.page, n_heads, rank,
                   _ptr(sink), _ptr(out), dtype_code(out.dtype), out.shape[1], scale, window, n,
                   self._stream())

    # -- windowed attention with pooled blocks; the delta rule --------------------------
    def qk_norm_rope_append(self, src, q_col, k_col, q_gamma, k_gamma, eps, freq, rot_dims,
                            amplitude, layout, kv, n_heads, q_out, write):
        """Per head: RMS norm (weights ``q_gamma`` / ``k_gamma`` over the head) and rotation by
        position of the queries and keys in the fp32 rows ``src``; queries to ``q_out``, keys to
        the K plane of ``kv`` and the keys as projected to its V plane (``write``)."""
        _check(src, "src", torch.float32, 2)
        _check(q_out, "q_out", None, 2)
        d, G = kv.head_dim, kv.n_kv_heads
        n = layout.n_rows
        if q_out.shape != (n, n_heads * d) or src.shape[0] < n or \
                src.shape[1] < max(q_col + n_heads * d, k_col + G * d) or \
                q_gamma.numel() != d or k_gamma.numel() != d or \
                (rot_dims and (freq is None or freq.numel() != rot_dims // 2)):
            raise KernelError("qk_norm_rope_append: shapes do not agree")
        self._call("nb_qk_norm_rope_append", _ptr(src), src.shape[1], q_col, k_col, _ptr(q_gamma),
                   _ptr(k_gamma), float(eps), _ptr(freq), int(rot_dims), float(amplitude),
                   _ptr(layout.row_slot), _ptr(layout.row_pos), _ptr(q_out), dtype_code(q_out.dtype),
                   _ptr(kv.k), _ptr(kv.v), dtype_code(kv.k.dtype), _ptr(kv.block_table),
                   kv.block_table.shape[1], kv.page, n_heads, G, d, 1 if write else 0, n,
                   self._stream())

    def qkv_norm_rope_append(self, src, q_col, k_col, v_col, q_gamma, k_gamma, eps, freq, rot_dims,
                             amplitude, layout, k_store, v_store, n_heads, value_dim, q_out, write):
        """Queries, keys and values of the fp32 rows ``src`` made ready: per head an optional RMS
        norm (``q_gamma`` / ``k_gamma`` or ``None``) and the rotation of the first ``rot_dims``
        numbers of queries and keys; queries to ``q_out``, keys to the K plane of ``k_store``,
        values (columns ``v_col ..``, heads of ``value_dim``) to the V plane of ``k_store`` when
        ``v_store`` is the same store, else to the one plane of ``v_store``."""
        _check(src, "src", torch.float32, 2)
        _check(q_out, "q_out", None, 2)
        d, G = k_store.head_dim, k_store.n_kv_heads
        n = layout.n_rows
        shared = v_store is k_store
        v_plane = k_store.v if shared else v_store.k
        if q_out.shape != (n, n_heads * d) or src.shape[0] < n or v_plane is None or \
                src.shape[1] < max(q_col + n_heads * d, k_col + G * d, v_col + G * value_dim) or \
                v_store.head_dim != value_dim or v_store.n_kv_heads != G or \
                (q_gamma is not None and (q_gamma.numel() != d or k_gamma.numel() != d)) or \
                (rot_dims and (freq is None or freq.numel() != rot_dims // 2)):
            raise KernelError("qkv_norm_rope_append: shapes do not agree")
        self._call("nb_qkv_norm_rope_append", _ptr(src), src.shape[1], q_col, k_col, v_col,
                   _ptr(q_gamma), _ptr(k_gamma), float(eps), _ptr(freq), int(rot_dims),
                   float(amplitude), _ptr(layout.row_slot), _ptr(layout.row_pos), _ptr(q_out),
                   dtype_code(q_out.dtype), _ptr(k_store.k), _ptr(v_plane),
                   dtype_code(k_store.k.dtype), _ptr(k_store.block_table),
                   k_store.block_table.shape[1], _ptr(v_store.block_table),
                   v_store.block_table.shape[1], k_store.page, n_heads, G, d, value_dim,
                   1 if write else 0, n, self._stream())

    def attention_masked(self, q, layout, k_store, v_store, n_heads, sink, out, scale, softcap=0.0,
                         window=0, keep_first=0, chunk=0, gate=None, gate_col=0):
        """Attention of the packed rows over ``k_store`` / ``v_store`` (as in
        :meth:`attention_capped`) where position ``i`` sees ``j <= i`` with ``i - j < window`` or
        ``j < keep_first`` (``window`` > 0), and only ``j`` of its own block of ``chunk`` positions
        (``chunk`` > 0).  ``gate``: fp32 rows with a logit per head at columns ``gate_col ..``;
        head ``h``'s result is multiplied by ``sigmoid`` of it."""
        _check(q, "q", None, 2)
        _check(out, "out", None, 2)
        n, d, dv = layout.n_rows, k_store.head_dim, v_store.head_dim
        shared = v_store is k_store
        if q.shape != (n, n_heads * d) or out.shape != (n, n_heads * dv) or \
                k_store.n_kv_heads != v_store.n_kv_heads or k_store.k.dtype != v_store.k.dtype or \
                (shared and k_store.v is None):
            raise KernelError("attention_masked: shapes do not agree")
        if sink is not None:
            _check(sink, "sink", torch.float32, 1)
            if sink.numel() != n_heads:
                raise KernelError("attention_masked: one sink per head")
        if gate is not None:
            _check(gate, "gate", torch.float32, 2)
            if gate.shape[0] < n or gate.shape[1] < gate_col + n_heads:
                raise KernelError("attention_masked: gate columns do not fit")
        look_back = window if window > 0 else chunk
        keeps = window > 0 and keep_first > 0
        code = dtype_code(q.dtype)
        if shared and q.dtype == k_store.k.dtype and layout.is_decode and \
                self.lib.nb_attention_decode_supported(code, d, n_heads, k_store.n_kv_heads, k_store.page) \
                and (q.dtype != torch.bfloat16 or q.shape[1] % 8 == 0):
            # one-token steps: the split decode kernel; kept first tokens are its last split, the
            # gate is applied where a row's sum divides its result
            pages = max(1, -(-layout.max_kv_len // k_store.page))
            if look_back > 0:
                pages = min(pages, (look_back + k_store.page - 1) // k_store.page + 1)
            n_splits = self._decode_splits(n * k_store.n_kv_heads, pages, k_store, q.dtype) + (1 if keeps else 0)
            acc, ml, counters = self._decode_scratch(q.device, n, n_heads, k_store.n_kv_heads, d, n_splits)
            self._call("nb_attention_decode_capped", _ptr(q), code, q.shape[1], 0,
                       _ptr(layout.row_slot), _ptr(layout.row_pos), _ptr(k_store.k), _ptr(k_store.v),
                       _ptr(k_store.block_table), k_store.block_table.shape[1], k_store.page, n_heads,
                       k_store.n_kv_heads, d, _ptr(out), dtype_code(out.dtype), out.shape[1],
                       float(scale), float(softcap or 0.0), _ptr(sink), int(window), int(keep_first),
                       int(chunk), _ptr(gate), gate.shape[1] if gate is not None else 0, int(gate_col),
                       n, n_splits, _ptr(acc), _ptr(ml), _ptr(counters), self._stream())
            return
        if shared and q.dtype == k_store.k.dtype and not layout.is_decode and self.use_tcgen05 \
                and scale > 0 and self.lib.nb_attention_prefill_tc_supported(
                    code, d, n_heads, k_store.n_kv_heads, k_store.page, q.shape[1], 0,
                    dtype_code(out.dtype), out.shape[1]):
            # prompts in bfloat16 with heads of 64 or 128: tcgen05 tiles of 128 rows; the pages a
            # tile reads are cut into runs when CTAs would idle, and kept first tokens that lie
            # before a tile's window are one more run
            if layout.n_rows > layout.n_tokens:
                out[layout.n_tokens:layout.n_rows].zero_()      # padding rows
            tiles = -(-layout.max_q_len // 128)
            ctas = tiles * n_heads * layout.n_seqs
            pages = -(-layout.max_kv_len // k_store.page)
            if look_back > 0:
                pages = min(pages, (look_back + 127) // k_store.page + 2)
            runs = 1
            if 2 * ctas <= PREFILL_TARGET_CTAS and pages >= 8:
                runs = min(4, PREFILL_TARGET_CTAS // ctas, pages // 4)
            per_run = -(-pages // runs)
            max_splits = runs + (1 if keeps else 0)
            part = counters = None
            if max_splits > 1:
                part, counters = self._prefill_scratch(q.device, ctas, max_splits, d)
            self._call("nb_attention_prefill_tc_masked", _ptr(q), code, q.shape[1], 0, q.shape[0],
                       _ptr(layout.cu_rows), _ptr(layout.seq_slot), _ptr(layout.seq_pos0),
                       _ptr(k_store.k), _ptr(k_store.v), k_store.k.shape[0], _ptr(k_store.block_table),
                       k_store.block_table.shape[1], k_store.page, n_heads, k_store.n_kv_heads, d,
                       _ptr(out), dtype_code(out.dtype), out.shape[1], float(scale),
                       float(softcap or 0.0), _ptr(sink), int(window), int(keep_first), int(chunk),
                       _ptr(gate), gate.shape[1] if gate is not None else 0, int(gate_col),
                       layout.n_seqs, layout.max_q_len, max_splits, per_run, _ptr(part),
                       _ptr(counters), 0, 0, 0, self._stream())
            return
        if shared and q.dtype == torch.bfloat16 and k_store.k.dtype == torch.bfloat16 \
                and not layout.is_decode and self.use_mma and self.lib.nb_attention_prefill_supported(
                    code, d, n_heads, k_store.n_kv_heads, k_store.page, q.shape[1], 0):
            # prompts in bfloat16 with other heads (16, 32, 48, 96; 64 and 128 when tcgen05 is
            # switched off): mma.sync tiles of 64 rows, the pages of kept first tokens walked
            # before the window's
            if layout.n_rows > layout.n_tokens:
                out[layout.n_tokens:layout.n_rows].zero_()      # padding rows
            self._call("nb_attention_prefill_masked", _ptr(q), q.shape[1], 0, _ptr(layout.cu_rows),
                       _ptr(layout.seq_slot), _ptr(layout.seq_pos0), _ptr(k_store.k), _ptr(k_store.v),
                       _ptr(k_store.block_table), k_store.block_table.shape[1], k_store.page, n_heads,
                       k_store.n_kv_heads, d, _ptr(sink), _ptr(out), dtype_code(out.dtype),
                       out.shape[1], float(scale), float(softcap or 0.0), int(window),
                       int(keep_first), int(chunk), _ptr(gate),
                       gate.shape[1] if gate is not None else 0, int(gate_col), layout.n_seqs,
                       layout.max_q_len, self._stream())
            return
        # any sizes and types, fp32 arithmetic: the 32-bit path, and what the kernels above leave
        v_plane = k_store.v if shared else v_store.k
        self._call("nb_attention_masked", _ptr(q), dtype_code(q.dtype), _ptr(layout.row_slot),
                   _ptr(layout.row_pos), _ptr(k_store.k), _ptr(k_store.block_table),
                   k_store.block_table.shape[1], _ptr(v_plane), _ptr(v_store.block_table),
                   v_store.block_table.shape[1], dtype_code(k_store.k.dtype), k_store.page, n_heads,
                   k_store.n_kv_heads, d, dv, _ptr(sink), _ptr(out), dtype_code(out.dtype),
                   float(scale), float(softcap or 0.0), int(window), int(keep_first), int(chunk),
                   _ptr(gate), gate.shape[1] if gate is not None else 0, int(gate_col), n,
                   self._stream())

    def pool_blocks(self, layout, kv, blocks, pool):
        """For every row that completes a block of ``pool`` tokens: the means of the block's keys
        and values in ``kv`` into entry ``pos // pool`` of the paged store ``blocks``."""
        if blocks.k.dtype != kv.k.dtype or blocks.head_dim != kv.head_dim or \
                blocks.n_kv_heads != kv.n_kv_heads or blocks.page != kv.page:
            raise KernelError("pool_blocks: the two stores differ in shape or type")
        self._call("nb_pool_blocks", _ptr(layout.row_slot), _ptr(layout.row_pos), _ptr(kv.k),
                   _ptr(kv.v), _ptr(kv.block_table), kv.block_table.shape[1], _ptr(blocks.k),
                   _ptr(blocks.v), _ptr(blocks.block_table), blocks.block_table.shape[1],
                   dtype_code(kv.k.dtype), kv.page, kv.n_kv_heads, kv.head_dim, int(pool),
                   layout.n_rows, self._stream())

    def attention_pooled(self, q, layout, kv, blocks, n_heads, sink, out, scale, window, pool):
        """Attention of the packed rows over the last ``window`` tokens of ``kv`` and the pooled
        blocks (``blocks``, or ``None``) that lie wholly before the window, with a sink."""
        _check(q, "q", None, 2)
        _check(out, "out", None, 2)
        n, d = layout.n_rows, kv.head_dim
        if q.shape != (n, n_heads * d) or out.shape != (n, n_heads * d):
            raise KernelError("attention_pooled: shapes do not agree")
        if sink is not None:
            _check(sink, "sink", torch.float32, 1)
        if self.use_mma and q.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16 \
                and self.lib.nb_attention_prefill_supported(1, d, n_heads, kv.n_kv_heads, kv.page,
                                                            q.shape[1], 0):
            # bfloat16 on the tensor cores (mma.sync), prompts and one-token steps alike: tiles
            # of 64 query rows, the pages of pooled blocks walked before the window's
            self._call("nb_attention_pooled_mma", _ptr(q), q.shape[1], 0, _ptr(layout.cu_rows),
                       _ptr(layout.seq_slot), _ptr(layout.seq_pos0), _ptr(kv.k), _ptr(kv.v),
                       _ptr(kv.block_table), kv.block_table.shape[1],
                       _ptr(blocks.k if blocks is not None else None),
                       _ptr(blocks.v if blocks is not None else None),
                       _ptr(blocks.block_table if blocks is not None else None),
                       blocks.block_table.shape[1] if blocks is not None else 0, kv.page, n_heads,
                       kv.n_kv_heads, d, _ptr(sink), _ptr(out), dtype_code(out.dtype), out.shape[1],
                       float(scale), int(window), int(pool), layout.n_seqs, layout.max_q_len,
                       self._stream())
            return
        self._call("nb_attention_pooled", _ptr(q), dtype_code(q.dtype), _ptr(layout.row_slot),
                   _ptr(layout.row_pos), _ptr(kv.k), _ptr(kv.v), _ptr(kv.block_table),
                   kv.block_table.shape[1], _ptr(blocks.k if blocks is not None else None),
                   _ptr(blocks.v if blocks is not None else None),
                   _ptr(blocks.block_table if blocks is not None else None),
                   blocks.block_table.shape[1] if blocks is not None else 0,
                   dtype_code(kv.k.dtype), kv.page, n_heads, kv.n_kv_heads, d, _ptr(sink), _ptr(out),
                   dtype_code(out.dtype), float(scale), int(window), int(pool), n, self._stream())

    def delta_rule(self, fused, col_r, col_k, col_v, col_g, col_a, decay_logits, a_bias, norm_w,
                   eps, decay_rate, key_eps, layout, state, n_heads, dim, out):
        """The generalized delta rule over each sequence's rows in order, from and into the
        sequences' state rows (``state``: fp32 ``[n_slots, n_heads * dim * dim]``); the heads'
        outputs normed, weighted and gated into ``out``."""
        _check(fused, "fused", torch.float32, 2)
        _check(decay_logits, "decay_logits", torch.float32, 2)
        _check(state, "state", torch.float32, 2)
        _check(out, "out", None, 2)
        n, hd = layout.n_rows, n_heads * dim
        if out.shape != (n, hd) or decay_logits.shape != (n, hd) or a_bias.numel() != hd or \
                norm_w.numel() != hd or state.shape[1] != hd * dim or \
                fused.shape[1] < max(col_r, col_k, col_v, col_g, col_a) + hd:
            raise KernelError("delta_rule: shapes do not agree")
        # the heads' outputs before their norm (the recurrence runs a head's columns in several
        # CTAs; the norm over the head is a pass of its own)
        o_raw = torch.empty((n, hd), device=out.device, dtype=torch.float32)
        self._call("nb_delta_rule", _ptr(fused), fused.shape[1], col_r, col_k, col_v, col_g, col_a,
                   _ptr(decay_logits), _ptr(a_bias), _ptr(norm_w), float(eps), float(decay_rate),
                   float(key_eps), _ptr(layout.cu_rows), _ptr(layout.seq_slot), _ptr(layout.row_slot),
                   _ptr(state), _ptr(o_raw), _ptr(out), dtype_code(out.dtype), n_heads, dim,
                   layout.n_seqs, n, self._stream())
        self.launches += 1

    # -- short convolutions, capped attention, linear recurrences ------------------------
    @staticmethod
    def _state_rows(state, n):
        """A mixer's part of the fixed-size state rows: fp32 ``[n_slots, n]``, rows ``stride(0)``
        floats apart (a view of some columns of the cache's rows)."""
        if state is None:
            return None
        if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or \
                state.shape[1] != n:
            raise KernelError(f"state rows: expected fp32 [slots, {n}] with unit column stride")
        return state

    def conv_rope_append(self, src, col0, w, taps, state, freq, rot_dims, layout, k_store,
                         v_store, n_heads, dv, q_out):
        """The short causal convolution (``w`` fp32 ``[channels, taps]``, or ``None`` for none)
        on the channels ``[queries | keys | values]`` of the fp32 rows ``src`` from column
        ``col0``, then the rotation by position of the queries' and keys' first ``rot_dims``
        numbers per head (neighbouring numbers paired); queries to ``q_out``, keys and values
        into the paged stores.  ``state``: the sequences' last ``taps - 1`` inputs, brought up
        to date for the next step."""
        _check(src, "src", torch.float32, 2)
        _check(q_out, "q_out", None, 2)
        d, G = k_store.head_dim, k_store.n_kv_heads
        C = n_heads * d + G * d + G * dv
        n = layout.n_rows
        taps = int(taps) if w is not None else 0
        if q_out.shape != (n, n_heads * d) or src.shape[0] < n or src.shape[1] < col0 + C or \
                v_store.head_dim != dv or v_store.n_kv_heads != G or \
                (w is not None and tuple(w.shape) != (C, taps)) or \
                (rot_dims and (freq is None or freq.numel() != rot_dims // 2)):
            raise KernelError("conv_rope_append: shapes do not agree")
        st = self._state_rows(state, (taps - 1) * C) if taps > 1 else None
        fused = 1 if layout.is_decode and layout.max_q_len == 1 else 0
        self._call("nb_conv_rope_append", _ptr(src), src.shape[1], col0, _ptr(w), taps, _ptr(st),
                   st.stride(0) if st is not None else 0, _ptr(layout.cu_rows),
                   _ptr(layout.seq_slot), _ptr(layout.seq_pos0), _ptr(freq), int(rot_dims),
                   _ptr(q_out), dtype_code(q_out.dtype), _ptr(k_store.k), _ptr(k_store.block_table),
                   k_store.block_table.shape[1],
                   _ptr(k_store.v if v_store is k_store else v_store.k), _ptr(v_store.block_table),
                   v_store.block_table.shape[1], dtype_code(k_store.k.dtype), k_store.page, n_heads,
                   G, d, dv, layout.n_seqs, layout.max_q_len, fused, self._stream())
        if taps > 1 and not fused:
            self._call("nb_conv_state_update", _ptr(src), src.shape[1], col0, taps, _ptr(st),
                       st.stride(0), _ptr(layout.cu_rows), _ptr(layout.seq_slot), C, layout.n_seqs,
                       self._stream())

    def conv_act(self, src, col0, w, bias, taps, act, state, layout, out_f32, out_act=None):
        """``out_f32 = act(conv(src[:, col0 : col0 + C]) + bias)`` per channel over time, the
        sequences' last ``taps - 1`` inputs kept in ``state``; ``out_act``: the same rows in the
        activation type (the next product's operand)."""
        _check(src, "src", torch.float32, 2)
        _check(out_f32, "out_f32", torch.float32, 2)
        n, C = out_f32.shape
        taps = int(taps) if w is not None else 0
        if n != layout.n_rows or src.shape[0] < n or src.shape[1] < col0 + C or \
                (w is not None and tuple(w.shape) != (C, taps)) or \
                (bias is not None and bias.numel() != C) or \
                (out_act is not None and out_act.shape != out_f32.shape):
            raise KernelError("conv_act: shapes do not agree")
        st = self._state_rows(state, (taps - 1) * C) if taps > 1 else None
        fused = 1 if layout.is_decode and layout.max_q_len == 1 else 0
        if out_act is not None and out_act.dtype == torch.float32:
            out_act = None          # the 32-bit rows are the operand
        self._call("nb_conv_act", _ptr(src), src.shape[1], col0, _ptr(w), _ptr(bias), taps, int(act),
                   _ptr(st), st.stride(0) if st is not None else 0, _ptr(layout.cu_rows),
                   _ptr(layout.seq_slot), C, _ptr(out_f32), _ptr(out_act),
                   dtype_code(out_act.dtype) if out_act is not None else 0, layout.n_seqs,
                   layout.max_q_len, fused, self._stream())
        if taps > 1 and not fused:
            self._call("nb_conv_state_update", _ptr(src), src.shape[1], col0, taps, _ptr(st),
                       st.stride(0), _ptr(layout.cu_rows), _ptr(layout.seq_slot), C, layout.n_seqs,
                       self._stream())

    def attention_capped(self, q, layout, k_store, v_store, n_heads, sink, out, scale, softcap):
        """Causal attention of the packed rows over the keys of ``k_store`` and the values of
        ``v_store`` (paged stores of one plane, head sizes ``d`` and ``dv``; or one store of two
        planes given twice, which the framework's attention kernels then read): scores ``scale *
        q . k``, with ``softcap`` > 0 replaced by ``softcap * tanh(score / softcap)``; ``sink``:
        fp32 ``[n_heads]`` logits of one more term of the softmax's denominator, or ``None``."""
        _check(q, "q", None, 2)
        _check(out, "out", None, 2)
        n, d, dv = layout.n_rows, k_store.head_dim, v_store.head_dim
        if q.shape != (n, n_heads * d) or out.shape != (n, n_heads * dv) or \
                k_store.n_kv_heads != v_store.n_kv_heads or k_store.k.dtype != v_store.k.dtype or \
                (v_store is k_store and k_store.v is None):
            raise KernelError("attention_capped: shapes do not agree")
        if sink is not None:
            _check(sink, "sink", torch.float32, 1)
            if sink.numel() != n_heads:
                raise KernelError("attention_capped: one sink per head")
        shared = v_store is k_store          # one store of two planes: keys and values of one size
        if shared and self.attention_takes(q, 0, layout, k_store, n_heads, out, scale):
            self.attention(q, 0, layout, k_store, n_heads, out, scale, 0, None, softcap, sink)
            return
        v_plane = k_store.v if shared else v_store.k
        self._call("nb_attention_capped", _ptr(q), dtype_code(q.dtype), _ptr(layout.row_slot),
                   _ptr(layout.row_pos), _ptr(k_store.k), _ptr(k_store.block_table),
                   k_store.block_table.shape[1], _ptr(v_plane), _ptr(v_store.block_table),
                   v_store.block_table.shape[1], dtype_code(k_store.k.dtype), k_store.page, n_heads,
                   k_store.n_kv_heads, d, dv, _ptr(sink), _ptr(out), dtype_code(out.dtype),
                   float(scale), float(softcap or 0.0), n, self._stream())

    def selective_scan(self, x, low, col_b, col_c, dt_lin, dt_bias, a_log, d_skip, z, z_col, state,
                       layout, n_state, out):
        """The selective scan over each sequence's rows in order, from and into the sequences'
        state rows (``[slots, inner * n_state]``): ``x`` the channels' inputs, ``low`` the rows
        holding B and C at columns ``col_b`` / ``col_c``, ``dt_lin`` the step sizes before bias
        and softplus, ``z`` (columns ``z_col ..``) the gates; all fp32."""
        for t, nm in ((x, "x"), (low, "low"), (dt_lin, "dt_lin"), (z, "z")):
            _check(t, nm, torch.float32, 2)
        _check(out, "out", None, 2)
        n, inner = layout.n_rows, x.shape[1]
        if out.shape != (n, inner) or dt_lin.shape != (n, inner) or x.shape[0] != n or \
                low.shape[1] < max(col_b, col_c) + n_state or z.shape[1] < z_col + inner or \
                dt_bias.numel() != inner or d_skip.numel() != inner or \
                tuple(a_log.shape) != (inner, n_state):
            raise KernelError("selective_scan: shapes do not agree")
        st = self._state_rows(state, inner * n_state)
        self._call("nb_selective_scan", _ptr(x), _ptr(low), low.shape[1], col_b, col_c, _ptr(dt_lin),
                   _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(z), z.shape[1], z_col, _ptr(st),
                   st.stride(0), _ptr(layout.cu_rows), _ptr(layout.seq_slot), inner, int(n_state),
                   _ptr(out), dtype_code(out.dtype), layout.n_seqs, self._stream())

    def linear_attention(self, fused, col_q, col_k, col_v, act, decay, state, layout, n_heads, d, dv,
                         out):
        """Per head ``S <- decay_h S + k v^T``, ``o = S^T q`` over each sequence's rows in order
        (``q, k, v`` = ``act`` of the columns of the fp32 rows ``fused``), from and into the
        state rows (``[slots, n_heads * d * dv]``); ``out``: fp32 ``[rows, n_heads * dv]``."""
        _check(fused, "fused", torch.float32, 2)
        _check(out, "out", torch.float32, 2)
        _check(decay, "decay", torch.float32, 1)
        n = layout.n_rows
        if out.shape != (n, n_heads * dv) or decay.numel() != n_heads or fused.shape[0] < n or \
                fused.shape[1] < max(col_q + n_heads * d, col_k + n_heads * d, col_v + n_heads * dv):
            raise KernelError("linear_attention: shapes do not agree")
        st = self._state_rows(state, n_heads * d * dv)
        self._call("nb_linear_attention", _ptr(fused), fused.shape[1], col_q, col_k, col_v, int(act),
                   _ptr(decay), _ptr(st), st.stride(0), _ptr(layout.cu_rows), _ptr(layout.seq_slot),
                   n_heads, d, dv, _ptr(out), layout.n_seqs, self._stream())

    def rmsnorm_gated(self, x, gamma, gate, gate_col, eps, out):
        """``out = x / sqrt(mean(x^2) + eps) * gamma * sigmoid(gate[:, gate_col : gate_col + d])``
        per fp32 row."""
        _check(x, "x", torch.float32, 2)
        _check(gate, "gate", torch.float32, 2)
        _check(gamma, "gamma", torch.float32, 1)
        _check(out, "out", None, 2)
        n, d = out.shape
        if x.shape != (n, d) or gamma.numel() != d or gate.shape[0] < n or gate.shape[1] < gate_col + d:
            raise KernelError("rmsnorm_gated: shapes do not agree")
        self._call("nb_rmsnorm_gated", _ptr(x), _ptr(gamma), _ptr(gate), gate.shape[1], gate_col,
                   _ptr(out), dtype_code(out.dtype), n, d, float(eps), self._stream())

    def rms_pair_add(self, a, gamma_a, b, gamma_b, eps, coef, residual, next_gamma=None,
                     next_eps=0.0, out_next=None):
        """``residual += coef * (rms-norm(a) * gamma_a + rms-norm(b) * gamma_b)`` per fp32 row,
        and in the same pass, where asked for, ``out_next = rms-norm(residual) * next_gamma``."""
        for t, nm in ((a, "a"), (b, "b"), (residual, "residual")):
            _check(t, nm, torch.float32, 2)
        n, d = residual.shape
        if a.shape != (n, d) or b.shape != (n, d) or gamma_a.numel() != d or gamma_b.numel() != d \
                or (out_next is not None and (out_next.shape != (n, d) or next_gamma is None
                                              or next_gamma.numel() != d)):
            raise KernelError("rms_pair_add: shapes do not agree")
        self._call("nb_rms_pair_add", _ptr(a), _ptr(gamma_a), _ptr(b), _ptr(gamma_b), float(eps),
                   float(coef), _ptr(residual), _ptr(next_gamma if out_next is not None else None),
                   float(next_eps), _ptr(out_next),
                   dtype_code(out_next.dtype) if out_next is not None else 0, n, d, self._stream())

    def glu_rows(self, x, gate_col, up_col, act, out, act_param=0.0):
        """``out[r, i] = act(x[r, gate_col + i]) * x[r, up_col + i]`` for fp32 rows ``x`` (or the
        combiner of ``ACT_SWISH_CLAMP`` with its bound ``act_param``)."""
        _check(x, "x", torch.float32, 2)
        _check(out, "out", None, 2)
        n, d = out.shape
        if x.shape[0] < n or x.shape[1] < max(gate_col, up_col) + d:
            raise KernelError("glu_rows: shapes do not agree")
        self._call("nb_glu_rows", _ptr(x), x.shape[1], gate_col, up_col, int(act), float(act_param),
                   _ptr(out), dtype_code(out.dtype), n, d, self._stream())

    def cast_cols(self, x, out, out_col):
        """``out[:, out_col : out_col + d] = x`` (fp32 rows into columns of rows of another type)."""
        _check(x, "x", torch.float32, 2)
        _check(out, "out", None, 2)
        n, d = x.shape
        if out.shape[0] != n or out.shape[1] < out_col + d:
            raise KernelError("cast_cols: shapes do not agree")
        self._call("nb_cast_cols", _ptr(x), _ptr(out), dtype_code(out.dtype), out.shape[1], out_col,
                   n, d, self._stream())

    # -- routed experts ---------------------------------------------------------------
    def moe_route(self, logits, col, n_experts, top, renormalize, layout, idx, weight):
        """Per row: softmax over the ``n_experts`` fp32 logits at columns ``col ..``, the ``top``
        largest (of equal scores the lower index) into ``idx`` / ``weight`` ``[rows, top]``."""
        _check(logits, "logits", torch.float32, 2)
        _check(idx, "idx", torch.int32, 2)
        _check(weight, "weight", torch.float32, 2)
        n = layout.n_rows
        if logits.shape[0] < n or idx.shape != (n, top) or weight.shape != (n, top):
            raise KernelError("moe_route: shapes do not agree")
        self._call("nb_moe_route", _ptr(logits), logits.shape[1], col, _ptr(layout.row_slot), n,
                   n_experts, top, 1 if renormalize else 0, _ptr(idx), _ptr(weight), self._stream())

    def moe_route_sigmoid(self, logits, col, bias, n_experts, top, n_groups, keep_groups, group_top,
                          renormalize, norm_eps, out_scale, layout, idx, weight):
        """Per row: ``s = sigmoid(logits)``; choice scores ``s + bias`` (``bias`` may be ``None``);
        with ``n_groups`` > 1 only experts of the ``keep_groups`` groups of neighbours with the
        largest sums of their ``group_top`` best choice scores can be chosen; the ``top`` best
        into ``idx``; ``weight`` = their ``s``, over ``(sum + norm_eps)`` if ``renormalize``,
        times ``out_scale``."""
        _check(logits, "logits", torch.float32, 2)
        _check(idx, "idx", torch.int32, 2)
        _check(weight, "weight", torch.float32, 2)
        if bias is not None:
            _check(bias, "bias", torch.float32, 1)
            if bias.numel() != n_experts:
                raise KernelError("moe_route_sigmoid: one bias per expert")
        n = layout.n_rows
        if logits.shape[0] < n or idx.shape != (n, top) or weight.shape != (n, top):
            raise KernelError("moe_route_sigmoid: shapes do not agree")
        self._call("nb_moe_route_sigmoid", _ptr(logits), logits.shape[1], col, _ptr(bias),
                   _ptr(layout.row_slot), n, n_experts, top, int(n_groups), int(keep_groups),
                   int(group_top), 1 if renormalize else 0, float(norm_eps), float(out_scale),
                   _ptr(idx), _ptr(weight), self._stream())

    def moe_group(self, idx, n_experts, offsets, order, place):
        """Group the (row, choice) pairs of ``idx`` by expert: ``offsets`` ``[n_experts + 1]``,
        ``order`` (place -> pair) and ``place`` (pair -> place, -1 for none), all int32."""
        for t, nm in ((idx, "idx"), (offsets, "offsets"), (order, "order"), (place, "place")):
            _check(t, nm, torch.int32)
        n_pairs = idx.numel()
        if offsets.numel() < n_experts + 1 or order.numel() < n_pairs or place.numel() < n_pairs:
            raise KernelError("moe_group: shapes do not agree")
        self._call("nb_moe_group", _ptr(idx), n_pairs, n_experts, _ptr(offsets), _ptr(order),
                   _ptr(place), self._stream())

    def moe_linear(self, x, order, row_div, offsets, w, w2, out, act=ACT_NONE, act_param=0.0):
        """A product per expert over its group: ``out[place] = x[row(place)] @ w[e].T``, or
        ``act(x @ w[e].T) * (x @ w2[e].T)`` with ``w2``; ``row(place) = order[place] // row_div``
        with ``order``, else ``place``.  ``w``, ``w2``: ``[n_experts, N, K]``.  ``act_param``: the
        number of a combiner that takes one (``ACT_SWISH_CLAMP``'s bound)."""
        _check(x, "x", None, 2)
        _check(w, "w", None, 3)
        _check(out, "out", None, 2)
        n_experts, N, K = w.shape
        if w2 is not None:
            _check(w2, "w2", w.dtype, 3)
            if w2.shape != w.shape:
                raise KernelError("moe_linear: the two weight sets differ in shape")
        if x.shape[1] != K or out.shape[1] != N or offsets.numel() < n_experts + 1:
            raise KernelError("moe_linear: shapes do not agree")
        n_places = out.shape[0]
        if self.use_mma and self.use_tcgen05 and n_places >= MOE_TC_MIN_PLACES \
                and out.dtype in (torch.bfloat16, torch.float32) and x.shape[1] % 8 == 0 \
                and self.lib.nb_moe_gemm_tc_supported(dtype_code(x.dtype), dtype_code(w.dtype),
                                                      n_places, n_experts, N, K):
            # many rows (a prompt): tcgen05 tiles of 128 places; the rows are brought into the
            # order of their places first, so that a tile is one TMA box
            xs = x
            if order is not None:
                xs = torch.empty((n_places, K), device=x.device, dtype=x.dtype)
                self._call("nb_moe_gather", _ptr(x), x.shape[1], _ptr(order), row_div, _ptr(offsets),
                           n_experts, _ptr(xs), n_places, K, self._stream())
            self._call("nb_moe_gemm_tc", _ptr(xs), xs.shape[0], _ptr(offsets), n_experts, n_places,
                       _ptr(w), _ptr(w2), _ptr(out), dtype_code(out.dtype), out.shape[1], N, K, act,
                       float(act_param), self._stream())
            return
        if self.use_mma and out.dtype in (torch.bfloat16, torch.float32) \
                and self.lib.nb_moe_gemm_mma_supported(dtype_code(x.dtype), dtype_code(w.dtype),
                                                       x.shape[1], K):
            self._call("nb_moe_gemm_mma", _ptr(x), x.shape[1], _ptr(order), row_div, _ptr(offsets),
                       n_experts, out.shape[0], _ptr(w), _ptr(w2), _ptr(out), dtype_code(out.dtype),
                       out.shape[1], N, K, act, float(act_param), self._stream())
            return
        self._call("nb_moe_gemm", _ptr(x), dtype_code(x.dtype), x.shape[1], _ptr(order), row_div,
                   _ptr(offsets), n_experts, out.shape[0], _ptr(w), _ptr(w2), dtype_code(w.dtype),
                   _ptr(out), dtype_code(out.dtype), out.shape[1], N, K, act, float(act_param),
                   self._stream())

    def moe_combine(self, y, place, weight, residual):
        """``residual[r] += sum_k weight[r, k] * y[place[r, k]]`` (fp32, ``k`` in order)."""
        _check(y, "y", torch.float32, 2)
        _check(place, "place", torch.int32)
        _check(weight, "weight", torch.float32, 2)
        _check(residual, "residual", torch.float32, 2)
        n, top = weight.shape
        if residual.shape[0] < n or residual.shape[1] != y.shape[1] or place.numel() < n * top:
            raise KernelError("moe_combine: shapes do not agree")
        self._call("nb_moe_combine", _ptr(y), y.shape[1], _ptr(place), _ptr(weight), top,
                   _ptr(residual), n, self._stream())

    def advance_decode(self, tokens, next_tokens, row_pos, row_slot):
        """tokens <- next_tokens, row_pos += 1 for live rows (between two decode steps)."""
        for t, n in ((tokens, "tokens"), (next_tokens, "next"), (row_pos, "row_pos"),
                     (row_slot, "row_slot")):
            _check(t, n, torch.int32, 1)
        self._call("nb_advance_decode", _ptr(tokens), _ptr(next_tokens), _ptr(row_pos),
                   _ptr(row_slot), (tokens.numel()), self._stream())

    # -- sampling ---------------------------------------------------------------------
    def argmax(self, logits, out):
        _check(logits, "logits", torch.float32, 2)
        _check(out, "out", torch.int32, 1)
        n, v = logits.shape
        n_ctas = min(32, max(1, v // 2048))
        if n_ctas > 1 and n * n_ctas <= 4096:
            s = self._argmax_scratch.get(logits.device)
            if s is None or s[0].numel() < n:
                s = (torch.zeros(max(n, 256), dtype=torch.int64, device=logits.device),
                     torch.zeros(max(n, 256), dtype=torch.int32, device=logits.device))
                self._argmax_scratch[logits.device] = s
            self._call("nb_argmax_split", _ptr(logits), n, v, _ptr(out), _ptr(s[0]),
                       _ptr(s[1]), n_ctas, self._stream())
            return
        self._call("nb_argmax", _ptr(logits), n, v, _ptr(out), self._stream())

    def sample_temperature(self, logits, temperature, u, out):
        _check(logits, "logits", torch.float32, 2)
        _check(u, "u", torch.float64, 1)
        _check(out, "out", torch.int32, 1)
        n, v = logits.shape
        self._call("nb_sample_temperature", _ptr(logits), n, v,
                   temperature, _ptr(u), _ptr(out), self._stream())

    def sample_top_k(self, logits, k, temperature, u, out):
        """Top-k sampling (no top-p) on the device: ``out[r]`` is drawn with ``u[r]`` among the
        row's ``k`` largest logits (ties at the k-th included); -1 marks a row with a NaN."""
        _check(logits, "logits", torch.float32, 2)
        _check(u, "u", torch.float64, 1)
        _check(out, "out", torch.int32, 1)
        n, v = logits.shape
        self._call("nb_sample_top_k", _ptr(logits), n, v, int(k), float(temperature), _ptr(u),
                   _ptr(out), self._stream())

    def top_p_max_k(self) -> int:
        """The largest top-k that :meth:`sample_top_p` takes together with top-p."""
        return int(self.lib.nb_sample_top_p_max_k())

    def sample_top_p(self, logits, k, top_p, temperature, u, out):
        """Top-p sampling (with top-k ``k``, 0 = off) on the device.  ``out[r]`` is the token,
        -1 for a row with a NaN, -2 for a row whose cut lies beyond the thousand largest logits
        (a flat distribution): those the caller settles on the host."""
        _check(logits, "logits", torch.float32, 2)
        _check(u, "u", torch.float64, 1)
        _check(out, "out", torch.int32, 1)
        n, v = logits.shape
        self._call("nb_sample_top_p", _ptr(logits), n, v, int(k), float(top_p), float(temperature),
                   _ptr(u), _ptr(out), self._stream())

    def top_candidates(self, logits, n_keep, temp):
        """The ``n_keep`` largest logits of every row with their indices (plus ties at the
        threshold, up to ``n_keep + 32``), the row maximum and the f64 sum of
        ``exp((x - max) / temp)`` over the row.  Returns ``(values [n, cap] f32, indices
        [n, cap] i32, counts [n] i32, stats [n, 2] f64)`` on the device; a count of -1 marks a
        row with a NaN, a count above ``cap`` ties that did not fit."""
        _check(logits, "logits", torch.float32, 2)
        n, v = logits.shape
        cap = n_keep + 32
        dev = logits.device
        vals = torch.empty((n, cap), dtype=torch.float32, device=dev)
        idx = torch.empty((n, cap), dtype=torch.int32, device=dev)
        counts = torch.empty(n, dtype=torch.int32, device=dev)
        stats = torch.empty((n, 2), dtype=torch.float64, device=dev)
        self._call("nb_top_candidates", _ptr(logits), n, v, n_keep, cap, float(temp), _ptr(vals),
                   _ptr(idx), _ptr(counts), _ptr(stats), self._stream())
        return vals, idx, counts, stats

    def history_append(self, history, history_len, tokens, row_slot):
        """history[r, history_len[r]] <- tokens[r], history_len[r] += 1 for live rows (a decode
        session's record of what each sequence has generated)."""
        _check(history, "history", torch.int32, 2)
        for t, n in ((history_len, "history_len"), (tokens, "tokens"), (row_slot, "row_slot")):
            _check(t, n, torch.int32, 1)
        self._call("nb_history_append", _ptr(history), history.shape[1], _ptr(history_len),
                   _ptr(tokens), _ptr(row_slot), tokens.numel(), self._stream())

    def repetition_penalty(self, logits, history, history_len, penalty):
        _check(logits, "logits", torch.float32, 2)
        _check(history, "history", torch.int32, 2)
        _check(history_len, "history_len", torch.int32, 1)
        n, v = logits.shape
        self._call("nb_repetition_penalty", _ptr(logits), n, v, _ptr(history),
                   history.shape[1], _ptr(history_len), penalty, self._stream())


_backend = None


def backend():
    """The installed backend; the CUDA library is loaded (and built) on first use."""
    global _backend
    if _backend is None:
        if not torch.cuda.is_available():
            raise KernelError(
                "no CUDA device: this library runs its models only through its sm_100a kernels "
                "and has no CPU path")
        _backend = CudaBackend()
    return _backend


def set_backend(b) -> None:
    """Install another backend object (tests of host logic) or ``None`` to reset."""
    global _backend
    _backend = b
