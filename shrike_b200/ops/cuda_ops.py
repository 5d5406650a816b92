"""The kernels, as one object the parts call.

Every method launches hand-written sm_100a code from `csrc/` through the C symbol
of its launcher, on torch's current stream, with raw device pointers.  There is no
CPU path and no library attention or model code: without a CUDA device, or when a
kernel cannot be built, construction fails.  Matrix products in bfloat16 run on this
package's tcgen05 kernel for up to 64 tokens (decoding) and go to cuBLAS through
`torch.mm` above that (Azimml/shrike's own GEMMs are cuBLAS calls through nn.Linear,
shrike/models/qwen.py:111-136); in float32 they run on this package's own FFMA
kernel, so the 32-bit path never touches a reduced-precision matrix mode.
"""

from __future__ import annotations

import ctypes

import torch

from . import build

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_c = ctypes
_P, _I, _F, _LL = _c.c_void_p, _c.c_int, _c.c_float, _c.c_longlong


class KernelError(RuntimeError):
    pass


class AttentionPlan:
    """What `CudaOps.attention_plan` decides for a batch shape."""

    __slots__ = ("has_single", "has_portions", "tc_portions", "splits", "cluster", "scratch", "arrivals",
                 "portion_splits", "portion_scratch")

    def __init__(self, has_single, has_portions, tc_portions, splits, cluster, scratch, arrivals,
                 portion_splits=1, portion_scratch=None):
        self.has_single, self.has_portions, self.tc_portions = has_single, has_portions, tc_portions
        self.splits, self.cluster, self.scratch, self.arrivals = splits, cluster, scratch, arrivals
        self.portion_splits, self.portion_scratch = portion_splits, portion_scratch   # the tensor-core portions kernel's key splits


def _ptr(tensor):
    return None if tensor is None else tensor.data_ptr()


_LIMITS = {
    "add_rmsnorm": "the row width must be at most 32768 (8192 when it is no multiple of 4)",
    "gather_add_rmsnorm": "the row width must be at most 32768 (8192 when it is no multiple of 4)",
    "norm_add": "the row width must be at most 32768 (8192 when it is no multiple of 4)",
    "gather_norm": "the row width must be at most 32768 (8192 when it is no multiple of 4)",
    "qk_norm_store": "a token's queries and keys together must fit an SM's shared memory (about 58,000 elements)",
    "latent_store": "the latent's rank must be at most 12288 and the row at least as wide as queries, latent and gates",
    "head_scale": "the head size must be a multiple of 4 and the array 16-byte aligned",
    "act_mul": "the activation must be one the kernels know and the run length divide the row",
    "gemm_tcgen05": "K must be a multiple of 8 and the operands 16-byte aligned",
    "tanh_norm": "at most four pending sums and two norms",
    "head_prep": "heads of at most 8192 elements, rotated dimensions even and at most the head's, the row at least as wide as q, k, v and gates",
    "matrix_memory_scan": "a positive gate cap, at most 65535 sequences and heads, the row at least as wide as q, k, v, gate and both gate columns, the state's heads at least dim * vdim + dim + 1 floats",
    "stream_norm": "1 to 8 streams, at most four pending sums, a row that fits an SM's shared memory",
    "short_conv": "1 to 32 taps, at most 65535 sequences, the convolved channels the projection's first columns",
    "gated_scan": "heads of at most 1024 rows, at most 65535 sequences, heads and runs of tokens, the row at least as wide as q, f and v, the state's heads at least dim * vdim floats",
    "route_top": "at most 1024 experts, 1 <= top <= experts, the weights [N, experts] or [N, experts + 1]",
    "act_mul_blocks": "experts * each columns at most, the rest the shared expert's, which needs the weights' last column",
    "paged_attention_bf16": "at most 65535 sequences and heads, heads a multiple of kv heads, at most 32 splits",
}


def _check(code: int, what: str):
    if code != 0:
        reason = f"bad argument ({_LIMITS[what]})" if code == -1 and what in _LIMITS else (
            "bad argument" if code == -1 else f"CUDA error {code}")
        raise KernelError(f"{what}: {reason}")


def _dense(tensor, dtype, what):
    if tensor.device.type != "cuda":
        raise KernelError(f"{what} must be on the GPU, is on {tensor.device}")
    if tensor.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, is {tensor.dtype}")
    if not tensor.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


class CudaOps:
    PORTION_SCRATCH_FLOATS = 32 << 20   # at most 128 MiB of partial rows for the split portions kernel

    def __init__(self, dtype: torch.dtype, device="cuda"):
        if dtype not in _DTYPE_CODE:
            raise KernelError(f"no kernels for {dtype}; bfloat16 and float32 are served")
        if not torch.cuda.is_available():
            raise KernelError("shrike_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
        self.dtype = dtype
        self.code = _DTYPE_CODE[dtype]
        self.device = torch.device(device)
        self.core = build.core_library()
        self._declare_core()
        self._attention = {}
        self.gemm_tc = None
        self.tensor_core_attention = True   # tcgen05 kernel for portions where the head and page sizes allow
        self.tensor_core_gemm_max_tokens = 64   # above this the library product is used
        self._partials = {}      # data_ptr of an output buffer -> its stack of K-split partial results
        # one host-visible word (of four): the first kernel whose bounded wait ran out, or that met
        # a row without a finite logit, leaves its code here; see `describe_status`
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        if dtype == torch.bfloat16:
            self.gemm_tc = build.tensor_core_gemm_library()
            self.gemm_tc.shrike_gemm_tc.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]
            self.gemm_tc.shrike_gemm_tc.restype = _I
            self.gemm_tc.shrike_gemm_tc_gated.argtypes = [_P, _P, _P, _I, _I, _I, _P, _P]
            self.gemm_tc.shrike_gemm_tc_gated.restype = _I
            self.gemm_tc.shrike_gemm_tc_gated_act.argtypes = [_P, _P, _P, _I, _I, _I, _I, _P, _P]
            self.gemm_tc.shrike_gemm_tc_gated_act.restype = _I
            self.gemm_tc.shrike_gemm_tc_gated_act_limit.argtypes = [_P, _P, _P, _I, _I, _I, _I, _F, _P, _P]
            self.gemm_tc.shrike_gemm_tc_gated_act_limit.restype = _I
            self.gemm_tc.shrike_gemm_tc_splits.argtypes = [_I, _I, _I]
            self.gemm_tc.shrike_gemm_tc_splits.restype = _I
        self._scratch = None     # partial results of split single-token attention
        self._sample_scratch = None  # per-slice winners of the sampling kernel
        self._arrivals = None    # per kv head: splits of single-token attention that have finished
        self._portion_scratch = None   # partial rows of the portions kernel when a query tile's keys are split
        self._portion_tiles = None
        self._memory_scratch = None   # what the matrix memory's chunk kernels hand from one launch to the next
        self._decay_scratch = None    # the same for the decayed linear attention: a state per run of tokens
        self._scan_scratch = None     # the gated recurrence's runs of tokens: each run's state, decay and first index
        self.portion_splits = 0  # 0: the kernel library's rule; n: that many key splits for portions (tests)
        self.generation = 0      # grows when the scratch moves
        self._held_stream = None
        self._layer_program = None   # the native per-layer issue, built on first use
        self.native_layers = True    # whole layers are issued by one native call where the parts allow it
        self.launches = 0        # launches of this package's own kernels
        self.library_calls = 0   # matrix products handed to cuBLAS
        # library matrix products keep float32 accumulation end to end: no TF32 for float32
        # inputs, no bfloat16 partial sums when a bfloat16 product is split along K
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    # ---- declarations -------------------------------------------------------
    def _declare_core(self):
        lib = self.core
        lib.shrike_embed.argtypes = [_P, _P, _I, _P, _I, _I, _I, _P, _I, _P]
        lib.shrike_add_rmsnorm.argtypes = [_P, _P, _I, _P, _P, _F, _P, _I, _I, _I, _I, _LL, _P]
        lib.shrike_silu_mul.argtypes = [_P, _P, _I, _I, _I, _I, _P]
        lib.shrike_rope_kv_write.argtypes = [_P] * 10 + [_I] * 5 + [_LL, _I, _LL, _P]
        lib.shrike_kv_write.argtypes = [_P] * 5 + [_I, _I, _I, _LL, _P]
        lib.shrike_gemm_fp32.argtypes = [_P, _P, _P, _P, _I, _I, _I, _P]
        lib.shrike_sample.argtypes = [_P, _P, _P, _P, _P, _P, _P, _I, _I, _P, _P]
        lib.shrike_embed_positions.argtypes = [_P, _P, _I, _P, _I, _I, _I, _P, _I, _P, _P, _I, _P]
        lib.shrike_act_mul.argtypes = [_P, _P, _I, _I, _I, _I, _I, _P]
        lib.shrike_norm_rows.argtypes = [_P, _P, _I, _I, _LL, _P, _P, _P, _F, _I, _P, _I, _I, _I, _P]
        lib.shrike_qk_norm_store.argtypes = [_P, _I, _LL, _P, _P, _F, _P, _F, _I, _P, _P, _P, _P] + [_I] * 6 + [_LL, _P]
        lib.shrike_latent_store.argtypes = [_P, _I, _LL, _P, _F, _P, _P, _P, _P] + [_I] * 7 + [_LL, _P]
        lib.shrike_head_scale.argtypes = [_P, _P, _I, _I, _I, _I, _P]
        lib.shrike_embed_scaled.argtypes = [_P, _P, _I, _P, _I, _I, _I, _P, _I, _P, _P, _I, _F, _P, _P]
        lib.shrike_act_mul_limit.argtypes = [_P, _P, _I, _I, _I, _I, _I, _F, _P]
        lib.shrike_tanh_norm.argtypes = [_P, _P, _P, _P, _P, _I, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _P]
        lib.shrike_head_prep.argtypes = [_P, _I, _LL, _I, _P, _P, _P, _I, _P, _P, _F, _P, _P, _P, _P, _P] + [_I] * 8 + [_P]
        lib.shrike_matrix_memory_scan.argtypes = [_P, _I, _LL, _I, _P, _P, _P, _P, _P, _P] + [_I] * 5 + [_F, _F, _F, _I, _I, _I, _P, _P, _P, _P, _P]
        lib.shrike_matrix_memory_out.argtypes = [_P, _P, _P, _I, _LL, _I, _I, _P, _F, _P, _I, _I, _I, _I, _P]
        lib.shrike_route_top.argtypes = [_P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P]
        lib.shrike_act_mul_blocks.argtypes = [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P]
        lib.shrike_matrix_memory_chunks.argtypes = [_I, _I]
        lib.shrike_matrix_memory_chunks.restype = _LL
        lib.shrike_decay_scan.argtypes = [_P, _I, _LL, _I, _P, _P, _P, _P, _P] + [_I] * 9 + [_P, _P]
        lib.shrike_decay_scan_chunks.argtypes = [_I, _I]
        lib.shrike_decay_scan_chunks.restype = _LL
        lib.shrike_norm_gate.argtypes = [_P, _P, _I, _LL, _I, _I, _P, _F, _P, _I, _I, _I, _P]
        lib.shrike_latent_rope_store.argtypes = [_P, _I, _LL, _I, _P, _F, _P, _P, _F, _P, _P, _P] + [_I] * 6 + [_LL, _P]
        lib.shrike_concat_cast.argtypes = [_P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _P]
        lib.shrike_stream_norm.argtypes = [_P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _F, _P, _I, _P, _P, _I, _I, _I, _P]
        lib.shrike_short_conv.argtypes = [_P, _I, _LL, _I, _P, _P, _P, _P, _P, _P, _P] + [_I] * 5 + [_P]
        lib.shrike_gated_scan.argtypes = [_P, _I, _LL, _I, _P, _P, _P, _P, _P, _P] + [_I] * 7 + [_P, _P, _P, _I, _I, _P]
        lib.shrike_gated_scan_runs.argtypes = [_I, _I, _I]
        lib.shrike_gated_scan_runs.restype = _LL
        lib.shrike_head_rms.argtypes = [_P, _P, _P, _I, _I, _I, _I, _F, _P]
        lib.shrike_head_prep_norms.argtypes = [_P, _I, _LL, _I, _P, _P, _P, _I, _P, _P, _F, _P, _P, _P, _P, _P] + [_I] * 10 + [_P]
        lib.shrike_route_top_scores.argtypes = [_P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P]
        lib.shrike_act_mul_blocks_at.argtypes = [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P]
        for name in ("shrike_decay_scan", "shrike_norm_gate", "shrike_latent_rope_store", "shrike_concat_cast",
                     "shrike_stream_norm", "shrike_short_conv", "shrike_gated_scan", "shrike_head_rms",
                     "shrike_head_prep_norms", "shrike_route_top_scores", "shrike_act_mul_blocks_at"):
            getattr(lib, name).restype = _I
        for name in ("shrike_embed_scaled", "shrike_act_mul_limit", "shrike_tanh_norm", "shrike_head_prep",
                     "shrike_matrix_memory_scan", "shrike_matrix_memory_out", "shrike_route_top", "shrike_act_mul_blocks"):
            getattr(lib, name).restype = _I
        lib.shrike_sample_slices.argtypes = [_I]
        lib.shrike_sample_slices.restype = _I
        for name in ("shrike_embed", "shrike_add_rmsnorm", "shrike_silu_mul", "shrike_rope_kv_write",
                     "shrike_kv_write", "shrike_gemm_fp32", "shrike_sample", "shrike_embed_positions", "shrike_act_mul",
                     "shrike_norm_rows", "shrike_qk_norm_store", "shrike_latent_store", "shrike_head_scale"):
            getattr(lib, name).restype = _I

    def _attention_lib(self, head_dim: int):
        lib = self._attention.get(head_dim)
        if lib is None:
            self.check_head_dim(head_dim)
            lib = build.attention_library(head_dim)
            lib.shrike_paged_attention_generic.argtypes = (
                [_P, _P, _P, _P, _I, _P, _P, _P] + [_I] * 6 + [_F, _I, _F, _P, _P, _P]
            )
            lib.shrike_paged_attention_generic.restype = _I
            lib.shrike_paged_attention_generic_sinks.argtypes = (
                [_P, _P, _P, _P, _I, _P, _P, _P] + [_I] * 6 + [_F, _I, _F, _P, _P, _P, _P]
            )
            lib.shrike_paged_attention_generic_sinks.restype = _I
            lib.shrike_paged_attention_generic_kept.argtypes = (
                [_P, _P, _P, _P, _I, _P, _P, _P] + [_I] * 6 + [_F, _I, _F, _P, _P, _I, _P, _P]
            )
            lib.shrike_paged_attention_generic_kept.restype = _I
            if head_dim <= build.TENSOR_CORE_HEAD_DIM:
                self._declare_tensor_core_attention(lib)
            self._attention[head_dim] = lib
        return lib

    @staticmethod
    def _declare_tensor_core_attention(lib):
        lib.shrike_paged_attention_bf16.argtypes = (
            [_P, _P, _P, _P, _I, _P, _P] + [_I] * 5 + [_F, _I, _P] + [_I] * 5 + [_P, _P, _P, _P]
        )
        lib.shrike_paged_attention_bf16.restype = _I
        lib.shrike_paged_attention_bf16_scores.argtypes = (
            [_P, _P, _P, _P, _I, _P, _P] + [_I] * 5 + [_F, _I, _P] + [_I] * 5 + [_P, _P, _P, _F, _P, _P]
        )
        lib.shrike_paged_attention_bf16_scores.restype = _I
        lib.shrike_paged_attention_bf16_sinks.argtypes = (
            [_P, _P, _P, _P, _I, _P, _P] + [_I] * 5 + [_F, _I, _P] + [_I] * 5 + [_P, _P, _P, _F, _P, _P, _P]
        )
        lib.shrike_paged_attention_bf16_sinks.restype = _I
        lib.shrike_paged_attention_bf16_kept.argtypes = (
            [_P, _P, _P, _P, _I, _P, _P] + [_I] * 5 + [_F, _I, _P] + [_I] * 5 + [_P, _P, _P, _F, _P, _P, _I, _P]
        )
        lib.shrike_paged_attention_bf16_kept.restype = _I
        lib.shrike_attention_single_token_pages.argtypes = [_I]
        lib.shrike_attention_single_token_pages.restype = None
        lib.shrike_attention_bf16_resident_ctas.restype = _I
        lib.shrike_attention_tc_available.restype = _I
        lib.shrike_paged_attention_tc_portions.argtypes = (
            [_P, _P, _P, _P, _I, _P, _P] + [_I] * 6 + [_F, _I, _P, _I, _I, _P, _I, _P, _I, _P, _P]
        )
        lib.shrike_paged_attention_tc_portions.restype = _I
        lib.shrike_paged_attention_tc_portions_scores.argtypes = (
            [_P, _P, _P, _P, _I, _P, _P] + [_I] * 6 + [_F, _I, _P, _I, _I, _P, _I, _P, _I, _P, _F, _P, _P]
        )
        lib.shrike_paged_attention_tc_portions_scores.restype = _I
        lib.shrike_paged_attention_tc_portions_sinks.argtypes = (
            [_P, _P, _P, _P, _I, _P, _P] + [_I] * 6 + [_F, _I, _P, _I, _I, _P, _I, _P, _I, _P, _F, _P, _P, _P]
        )
        lib.shrike_paged_attention_tc_portions_sinks.restype = _I
        lib.shrike_paged_attention_tc_portions_kept.argtypes = (
            [_P, _P, _P, _P, _I, _P, _P] + [_I] * 6 + [_F, _I, _P, _I, _I, _P, _I, _P, _I, _P, _F, _P, _P, _I, _P]
        )
        lib.shrike_paged_attention_tc_portions_kept.restype = _I
        lib.shrike_attention_tc_portions_rows.restype = _I
        lib.shrike_attention_tc_portions_splits.argtypes = [_I, _I, _I, _I, _I]
        lib.shrike_attention_tc_portions_splits.restype = _I
        lib.shrike_attention_tc_portions_scratch_floats.argtypes = [_I, _I, _I]
        lib.shrike_attention_tc_portions_scratch_floats.restype = _LL

    def _stream(self):
        return self._held_stream if self._held_stream is not None else torch.cuda.current_stream().cuda_stream

    def hold_stream(self, hold: bool) -> None:
        """Between `hold_stream(True)` and `hold_stream(False)` every launch goes to the stream
        that was current at the first call, looked up once: asking torch for the current stream
        costs more than a launch.  The step function brackets a forward pass with it."""
        self._held_stream = torch.cuda.current_stream().cuda_stream if hold else None

    def check_head_dim(self, head_dim: int):
        if head_dim % 16 or not 16 <= head_dim <= 1024:
            raise KernelError(
                f"head size {head_dim} is not served: the attention kernels take multiples of 16 from 16 to 1024 "
                "(the tensor-core ones up to 256)"
            )

    def layer_program(self):
        """The native per-layer issue (`ops/layer_program.py`), or None when it is switched off."""
        if not self.native_layers or self.dtype != torch.bfloat16:
            return None
        if self._layer_program is None:
            from .layer_program import LayerProgram

            self._layer_program = LayerProgram(self)
        return self._layer_program

    # ---- kernels ------------------------------------------------------------
    def embed(self, ids, table, out, previous=None, position_table=None, positions=None, scale=1.0, keep=None):
        """Rows of `table`, each times `scale`, into the float32 residual.  An id of -1 - r is replaced on
        the device by `previous[r]` (int32: the tokens the step before drew).  With `position_table`
        ([max positions, width], the type of `table`) the row of each token's position is added.
        `keep` (float32, the shape of `out`) receives a second copy of the result."""
        _dense(ids, torch.int32, "token ids")
        _dense(out, torch.float32, "residual")
        n, width = out.shape
        if previous is not None:
            _dense(previous, torch.int32, "previous tokens")
        if position_table is not None:
            _dense(position_table, table.dtype, "position table")
            _dense(positions, torch.int32, "positions")
            if position_table.shape[1] != width:
                raise KernelError("the position table's rows must be as wide as the residual")
        if keep is not None:
            _dense(keep, torch.float32, "kept embedding")
            if tuple(keep.shape) != tuple(out.shape):
                raise KernelError("the kept copy must have the residual's shape")
        self.launches += 1
        _check(self.core.shrike_embed_scaled(
            _ptr(ids), _ptr(table), _DTYPE_CODE[table.dtype], _ptr(out), n, width, table.shape[0], _ptr(previous),
            0 if previous is None else previous.numel(), _ptr(position_table), _ptr(positions),
            0 if position_table is None else position_table.shape[0], float(scale), _ptr(keep), self._stream()), "embed")

    @staticmethod
    def _stack(delta):
        """(partials, stride in elements) of a [N, W] array or a [P, N, W] stack of partial sums."""
        if delta is None or delta.dim() == 2:
            return 1, 0
        return delta.shape[0], delta.stride(0)

    def add_rmsnorm(self, resid, delta, weight, eps, out):
        """resid += delta (a [N, W] array, or a [P, N, W] stack added in order); out = norm(resid) * weight."""
        _dense(resid, torch.float32, "residual")
        _dense(weight, torch.float32, "norm weight")
        n, width = resid.shape
        code = -1 if delta is None else _DTYPE_CODE[delta.dtype]
        partials, stride = self._stack(delta)
        self.launches += 1
        _check(self.core.shrike_add_rmsnorm(_ptr(resid), _ptr(delta), code, None, _ptr(weight), eps, _ptr(out),
                                            _DTYPE_CODE[out.dtype], n, width, partials, stride, self._stream()),
               "add_rmsnorm")

    def gather_add_rmsnorm(self, resid, delta, rows, weight, eps, out):
        _dense(resid, torch.float32, "residual")
        _dense(rows, torch.int32, "rows")
        width = resid.shape[1]
        code = -1 if delta is None else _DTYPE_CODE[delta.dtype]
        partials, stride = self._stack(delta)
        self.launches += 1
        _check(self.core.shrike_add_rmsnorm(_ptr(resid), _ptr(delta), code, _ptr(rows), _ptr(weight), eps,
                                            _ptr(out), _DTYPE_CODE[out.dtype], rows.shape[0], width, partials,
                                            stride, self._stream()), "gather_add_rmsnorm")

    def norm_add(self, resid, branch, weight, bias, eps, out, layer_norm=True):
        """resid += norm(branch) (float32 sum), for a branch [N, W] or a [P, N, W] stack of partial sums;
        `out` (may be None) gets the new residual in its own type.  `branch` None: only that cast.
        norm: layer norm with the variance as the mean squared deviation (`layer_norm`), else RMS."""
        _dense(resid, torch.float32, "residual")
        n, width = resid.shape
        code = -1 if branch is None else _DTYPE_CODE[branch.dtype]
        partials, stride = self._stack(branch)
        self.launches += 1
        _check(self.core.shrike_norm_rows(
            _ptr(resid), _ptr(branch), code, partials, stride, None, _ptr(weight), _ptr(bias), eps, int(layer_norm),
            _ptr(out), -1 if out is None else _DTYPE_CODE[out.dtype], n, width, self._stream()), "norm_add")

    def gather_norm(self, resid, rows, weight, bias, eps, out, layer_norm=True):
        """out[r] = norm(resid[rows[r]]): the final norm on the wanted rows only."""
        _dense(resid, torch.float32, "residual")
        _dense(rows, torch.int32, "rows")
        self.launches += 1
        _check(self.core.shrike_norm_rows(
            _ptr(resid), None, -1, 1, 0, _ptr(rows), _ptr(weight), _ptr(bias), eps, int(layer_norm),
            _ptr(out), _DTYPE_CODE[out.dtype], rows.shape[0], resid.shape[1], self._stream()), "gather_norm")

    def qk_norm_store(self, qk, q_weight, k_weight, eps, positions, temperature, q_out, keys, values, slots,
                      num_heads, num_kv_heads, dim, padded):
        """Queries and keys of a fused q|k projection ([N, (H + G) D] float32 or a K-split stack): each
        divided by its root mean square over the WHOLE projection and scaled by its weight (None: left
        as projected), the query times 1 + coef * ln(floor((p + 1) / every) + 1) for `temperature`
        (coef, every) at position p; queries to `q_out` [N, H * padded], keys to the key pages and the
        keys as projected to the value pages, heads `padded` elements apart (padding zeroed)."""
        _dense(qk, torch.float32, "q|k projection")
        _dense(q_out, self.dtype, "q")
        partials, stride = self._stack(qk)
        num_slots = 0
        if keys is not None:
            _dense(keys, self.dtype, "key cache")
            _dense(values, self.dtype, "value cache")
            num_slots = keys.shape[0] * keys.shape[1]
        coef, every = temperature if temperature is not None else (0.0, 0)
        self.launches += 1
        _check(self.core.shrike_qk_norm_store(
            _ptr(qk), partials, stride, _ptr(q_weight), _ptr(k_weight), eps, _ptr(positions), coef, every, _ptr(q_out),
            _ptr(keys), _ptr(values), _ptr(slots), self.code, qk.shape[-2], num_heads, num_kv_heads, dim, padded,
            num_slots, self._stream()), "qk_norm_store")

    def latent_store(self, fused, latent_weight, eps, q_out, latents, slots, gate_out, q_width, rank, padded, gates):
        """Splits a fused q|latent|gate projection ([N, at least q_width + rank + gates] float32 or a K-split
        stack; further columns are padding): queries cast to `q_out`, the latent divided by its root mean square and scaled by
        `latent_weight` into the latent pages (`padded` elements a token), sigmoid of the gate columns
        to `gate_out` (float32).  rank 0: no latent of its own; gates 0: no gate."""
        _dense(fused, torch.float32, "fused projection")
        _dense(q_out, self.dtype, "q")
        partials, stride = self._stack(fused)
        num_slots = 0
        if latents is not None:
            _dense(latents, self.dtype, "latent cache")
            num_slots = latents.shape[0] * latents.shape[1]
        self.launches += 1
        _check(self.core.shrike_latent_store(
            _ptr(fused), partials, stride, _ptr(latent_weight), eps, _ptr(q_out), _ptr(latents), _ptr(slots),
            _ptr(gate_out), self.code, fused.shape[-2], q_width, rank, padded, gates, fused.shape[-1], num_slots,
            self._stream()),
            "latent_store")

    def head_scale(self, x, gate, heads, dim):
        """x[n, h, :] *= gate[n, h] in place (gate float32 [N, heads])."""
        _dense(x, self.dtype, "head outputs")
        _dense(gate, torch.float32, "gate")
        self.launches += 1
        _check(self.core.shrike_head_scale(_ptr(x), _ptr(gate), self.code, x.shape[0], heads, dim, self._stream()),
               "head_scale")

    def linear(self, x, w, out, bias=None, allow_partials=False):
        """x[N, K] @ w[O, K]^T (+ bias) into `out` [N, O] (float32 or the activation type).

        Returns the array to consume: `out`, or, when `allow_partials` and the product was
        split along K, a float32 stack [P, N, O] whose sum over P is the result (the
        norm and rotary kernels add such stacks themselves)."""
        n, k = x.shape
        o = w.shape[0]
        if w.shape[1] != k or tuple(out.shape) != (n, o):
            raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
        if self.dtype == torch.float32:
            self.launches += 1
            _dense(x, torch.float32, "linear input")
            _dense(w, torch.float32, "linear weight")
            _dense(out, torch.float32, "linear output")
            _check(self.core.shrike_gemm_fp32(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), n, o, k, self._stream()),
                   "gemm_fp32")
            return out
        _dense(x, torch.bfloat16, "linear input")
        _dense(w, torch.bfloat16, "linear weight")
        if self.gemm_tc is not None and n <= self.tensor_core_gemm_max_tokens and k % 8 == 0:
            _dense(out, out.dtype, "linear output")
            splits, target = 1, out
            if allow_partials and out.dtype == torch.float32:
                splits = self.gemm_tc.shrike_gemm_tc_splits(n, o, k)
                if splits > 1:
                    target = self._partial_stack(out, splits)
            self.launches += 1
            _check(self.gemm_tc.shrike_gemm_tc(_ptr(x), _ptr(w), _ptr(bias), _ptr(target), _DTYPE_CODE[out.dtype],
                                               n, o, k, splits, _ptr(self.status), self._stream()), "gemm_tcgen05")
            return target
        self.library_calls += 1
        if out.dtype == torch.float32:
            torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
        else:
            torch.mm(x, w.t(), out=out)
        if bias is not None:
            out.add_(bias)
        return out

    def _partial_stack(self, out, splits):
        """The float32 [splits, N, O] stack that belongs to the output buffer `out`."""
        n, o = out.shape
        key = out.data_ptr()
        held = self._partials.get(key)
        need = splits * n * o
        if held is None or held.numel() < need:
            capacity = max(need, 16 * self.tensor_core_gemm_max_tokens * o)
            held = torch.empty(capacity, dtype=torch.float32, device=self.device)
            self._partials[key] = held
            self.generation += 1
        return held[:need].view(splits, n, o)

    def adopt_status(self, word: torch.Tensor) -> None:
        """Makes `word` (int32 [4] on the device, zeroed) the status word the kernels write, so that
        the step function can bring it to the host in the same copy as a step's drawn tokens.  To be
        called before the first launch: launch sequences that were captured keep the old address."""
        if word.dtype != torch.int32 or word.numel() < 4 or word.device != self.status.device:
            raise KernelError("the status word must be four int32 on the kernels' device")
        word.zero_()
        self.status = word
        self.generation += 1

    @staticmethod
    def describe_status(code: int) -> str:
        """What a nonzero status word means: which kernel gave up, and where."""
        roles = {
            1: "gemm_tcgen05: the TMA producer's wait for a free stage ran out",
            2: "gemm_tcgen05: the MMA issuer's wait for a loaded stage ran out",
            3: "gemm_tcgen05: the epilogue's wait for the accumulator ran out",
            4: "gemm_tcgen05: copies still in flight after an aborted wait",
            11: "attention_tcgen05 (portions): the loader's wait for a free key/value stage ran out",
            12: "attention_tcgen05 (portions): the MMA issuer's wait ran out",
            13: "attention_tcgen05 (portions): a softmax thread's wait ran out",
            14: "attention_tcgen05 (portions): copies still in flight after an aborted wait",
            15: "attention_tcgen05 (portions): shared memory was not aligned as the tiles need",
            21: "attention_bf16 (single tokens, by pages): the wait for a page's tile ran out",
            22: "attention_bf16 (single tokens, by pages): shared memory was not aligned as the tiles need",
            31: "sampling: a row of logits had no finite element (NaN logits); token 0 was returned for it",
        }
        return roles.get(code, f"unknown status code {code}")

    def raise_status(self, code: int):
        """Clears the status word (and the counters an aborted kernel may have left half-way) and
        raises: the results of the step that set `code` are not valid."""
        self.status.zero_()
        if self._arrivals is not None:
            self._arrivals.zero_()
        raise KernelError(f"{self.describe_status(code)}; the results of that step are not valid")

    def check_status(self):
        """Raises when a kernel left a code in the status word (reads one word from the device)."""
        code = int(self.status[0].item())
        if code:
            self.raise_status(code)

    def rope_kv_write(self, qkv, bias, positions, inv_freq, q_out, keys, values, slots,
                      num_heads, num_kv_heads, head_dim, k_out=None, v_out=None):
        """Bias, rotation and cache store of a fused q/k/v projection ([N, W] or a K-split stack).
        `positions`, `slots`, `bias` and `inv_freq` are read while the kernels launched before may
        still run (the angles are formed meanwhile): they must be the step's metadata or
        parameters, not something a kernel of this step computes."""
        _dense(qkv, torch.float32, "qkv")
        _dense(q_out, self.dtype, "q")
        partials, stride = self._stack(qkv)
        n = qkv.shape[-2]
        num_slots = 0
        if keys is not None:
            _dense(keys, self.dtype, "key cache")
            _dense(values, self.dtype, "value cache")
            num_slots = keys.shape[0] * keys.shape[1]
        self.launches += 1
        _check(self.core.shrike_rope_kv_write(
            _ptr(qkv), _ptr(bias), _ptr(positions), _ptr(inv_freq), _ptr(q_out), _ptr(keys), _ptr(values),
            _ptr(slots), _ptr(k_out), _ptr(v_out), self.code, n, num_heads, num_kv_heads, head_dim,
            num_slots, partials, stride, self._stream()), "rope_kv_write")

    def kv_write(self, k_new, v_new, keys, values, slots):
        _dense(keys, self.dtype, "key cache")
        n, kv_width = k_new.shape
        self.launches += 1
        _check(self.core.shrike_kv_write(_ptr(k_new), _ptr(v_new), _ptr(keys), _ptr(values), _ptr(slots),
                                         self.code, n, kv_width, keys.shape[0] * keys.shape[1],
                                         self._stream()), "kv_write")

    def paged_attention(self, q, keys, values, block_table, q_start, ctx_len, seq_of_token,
                        num_heads, num_kv_heads, head_dim, scale, window, out,
                        max_q_len=0, max_ctx_len=0, min_q_len=0, q_lens=None, softcap=None, slopes=None, chunk=None,
                        sinks=None, keep_first=0):
        """Attention of the batch's new tokens over the paged cache.  `window`: a query sees the `window`
        latest keys.  `chunk` (instead of a window): a query at position p sees key j <= p only when
        floor(p / chunk) = floor(j / chunk).  `max_q_len` and
        `min_q_len` are the longest and shortest entry of the batch (0: not known); `q_lens`, every
        entry's length (host list), lets the portions kernel launch exactly the CTAs it needs.
        `softcap` (a positive number) and `slopes` (float32 [num_heads]) change a score
        s = scale * q.k, in this order: s <- softcap * tanh(s / softcap), then
        s <- s - slopes[head] * (query position - key position).  `sinks` (float32 [num_heads]): exp(sinks[head])
        is one more term of every softmax's denominator: a weight that goes to nothing (the raw number, without `scale`).
        `keep_first` (with a window): the sequence's first `keep_first` keys stay visible to every later query."""
        _dense(q, self.dtype, "q")
        if sinks is not None:
            _dense(sinks, torch.float32, "softmax sinks")
            if sinks.numel() != num_heads:
                raise KernelError("one softmax sink per query head")
        _dense(keys, self.dtype, "key cache")
        _dense(values, self.dtype, "value cache")
        _dense(block_table, torch.int32, "block table")
        if keys.shape[2] != num_kv_heads or keys.shape[3] != head_dim:
            raise KernelError(f"key cache {tuple(keys.shape)} does not fit {num_kv_heads} heads of {head_dim}")
        lib = self._attention_lib(head_dim)
        num_seqs, max_blocks = block_table.shape
        page_size, num_pages = keys.shape[1], keys.shape[0]
        if chunk:
            if window:
                raise KernelError("attention takes a window or a chunk, not both")
            window = -int(chunk)   # the kernels' one number: > 0 a window, < 0 runs of that many positions
        keep_first = int(keep_first) if window and window > 0 else 0
        if self.dtype == torch.float32 or head_dim > build.TENSOR_CORE_HEAD_DIM:
            self.launches += 1
            _check(lib.shrike_paged_attention_generic_kept(
                _ptr(q), _ptr(keys), _ptr(values), _ptr(block_table), max_blocks, _ptr(q_start),
                _ptr(ctx_len), _ptr(seq_of_token), self.code, q.shape[0], num_heads, num_kv_heads,
                page_size, num_pages, scale, window or 0, softcap or 0.0, _ptr(slopes), _ptr(sinks), keep_first, _ptr(out),
                self._stream()), "paged_attention")
            return
        if slopes is not None:
            _dense(slopes, torch.float32, "distance slopes")
            if slopes.numel() != num_heads:
                raise KernelError("one distance slope per query head")
        plan = self.attention_plan(num_heads, num_kv_heads, head_dim, num_seqs, max_blocks, page_size, max_q_len, min_q_len,
                                   q.shape[0], q_lens, keep_first=keep_first)
        self.launches += plan.has_single + plan.has_portions + (1 if plan.portion_splits > 1 else 0)
        has_portions = plan.has_portions
        if plan.tc_portions:
            _check(lib.shrike_paged_attention_tc_portions_kept(
                _ptr(q), _ptr(keys), _ptr(values), _ptr(block_table), max_blocks, _ptr(q_start), _ptr(ctx_len),
                q.shape[0], num_seqs, num_heads, num_kv_heads, page_size, num_pages, scale, window or 0, _ptr(out),
                plan.has_single, max_q_len, _ptr(self.status), plan.portion_splits, _ptr(plan.portion_scratch),
                self.portion_tiles(q_lens, plan.has_single, lib.shrike_attention_tc_portions_rows()), _ptr(seq_of_token),
                softcap or 0.0, _ptr(slopes), _ptr(sinks), keep_first, self._stream()), "paged_attention_tc_portions")
            has_portions = 0
            if not plan.has_single:
                return
        _check(lib.shrike_paged_attention_bf16_kept(
            _ptr(q), _ptr(keys), _ptr(values), _ptr(block_table), max_blocks, _ptr(q_start), _ptr(ctx_len),
            num_seqs, num_heads, num_kv_heads, page_size, num_pages, scale, window or 0, _ptr(out),
            plan.has_single, has_portions, max_q_len, plan.splits, plan.cluster, _ptr(plan.scratch), _ptr(plan.arrivals),
            _ptr(self.status), softcap or 0.0, _ptr(slopes), _ptr(sinks), keep_first, self._stream()),
            "paged_attention_bf16")

    def portion_tiles(self, q_lens, skip_single, rows) -> int:
        """Query tiles of `rows` rows that the batch's portions make; 0 when the lengths are not known."""
        if q_lens is None:
            return 0
        held = self._portion_tiles
        if held is not None and held[0] is q_lens and held[1] == (skip_single, rows):
            return held[2]
        tiles = sum(-(-q // rows) for q in q_lens if q > 1 or not skip_single)
        self._portion_tiles = (q_lens, (skip_single, rows), tiles)
        return tiles

    def attention_plan(self, num_heads, num_kv_heads, head_dim, num_seqs, max_blocks, page_size, max_q_len, min_q_len,
                       num_tokens=0, q_lens=None, keep_first=0):
        """How a bfloat16 batch's attention is cut: which kernels run (single tokens, portions, the
        tensor-core form of the latter), the key splits and clusters of the single-token kernel, the
        key splits of the portions kernel, and their scratch.  A function of the batch's shape alone."""
        if max_q_len < 1:
            raise KernelError("paged_attention in bfloat16 needs max_q_len, the longest entry of the batch")
        lib = self._attention_lib(head_dim)
        has_single = min_q_len <= 1
        has_portions = max_q_len > 1
        splits, cluster, scratch, arrivals = 1, 1, None, None
        if has_single:
            row_tiles = -(-(num_heads // num_kv_heads) // 16)
            tiles = max(1, -(-(max_blocks * page_size) // 64))
            resident = lib.shrike_attention_bf16_resident_ctas()
            splits, cluster = self.single_token_splits(tiles, num_seqs * num_kv_heads * row_tiles, resident)
            need = num_seqs * num_heads * (splits // cluster) * (head_dim + 2)
            if self._scratch is None or self._scratch.numel() < need:
                self._scratch = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=self.device)
                self.generation += 1
            groups = num_seqs * num_kv_heads * row_tiles
            if self._arrivals is None or self._arrivals.numel() < groups:
                self._arrivals = torch.zeros(max(groups, 4096), dtype=torch.int32, device=self.device)
                self.generation += 1
            scratch, arrivals = self._scratch, self._arrivals
        tc_portions = bool(has_portions and self.tensor_core_attention and lib.shrike_attention_tc_available()
                           and page_size in (8, 16, 32, 64))
        portion_splits, portion_scratch = 1, None
        if tc_portions and num_tokens > 0:
            tiles = self.portion_tiles(q_lens, has_single, lib.shrike_attention_tc_portions_rows())
            portion_splits = self.portion_splits or lib.shrike_attention_tc_portions_splits(
                num_tokens, num_heads, max_blocks, page_size, tiles)
            kept = 1 if keep_first else 0   # kept first keys are one more split of their own, behind the window's
            need = lib.shrike_attention_tc_portions_scratch_floats(num_tokens, num_heads, portion_splits + kept)
            if need > self.PORTION_SCRATCH_FLOATS:   # bound the scratch: fewer splits, never a refusal
                portion_splits = max(1, (portion_splits + kept) * self.PORTION_SCRATCH_FLOATS // need - kept)
                need = lib.shrike_attention_tc_portions_scratch_floats(num_tokens, num_heads, portion_splits + kept)
            portion_splits += kept
            if portion_splits > 1:
                if self._portion_scratch is None or self._portion_scratch.numel() < need:
                    self._portion_scratch = torch.empty(max(need, 1 << 22), dtype=torch.float32, device=self.device)
                    self.generation += 1
                portion_scratch = self._portion_scratch
        return AttentionPlan(int(has_single), int(has_portions), int(tc_portions), splits, cluster, scratch, arrivals,
                             portion_splits, portion_scratch)

    @staticmethod
    def single_token_splits(tiles: int, groups: int, resident: int):
        """(splits, cluster) for single-token attention over `tiles` 64-key tiles of `groups`
        (sequence, kv head) pairs when `resident` CTAs fit the GPU at once.

        Up to eight splits may form a thread-block cluster and add up on chip.  That is the
        quickest way while the clusters fill no more than two thirds of the GPU; a fuller grid
        of clusters starts late (a cluster needs all its places free in one part of the chip
        at once, while the kernel before it is still leaving), and the splits then meet in
        global memory instead, eight partials to a round trip.  Long contexts take several
        clusters per pair, whose partials meet in global memory too."""
        want = max(1, min(tiles, resident // max(1, groups)))
        cluster = 1
        while cluster * 2 <= min(want, 8):
            cluster *= 2
        if cluster == 8 and groups * 8 * 3 > resident * 2:
            return min(want, 32) // 8 * 8, 1
        if tiles <= 4 * cluster or want < 2 * cluster:
            return cluster, cluster
        return min(want // cluster * cluster, 32 * cluster), cluster

    ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}   # the codes the kernels take

    def silu_mul(self, gate_up, out, block=0):
        """out = silu(gate) * up; see `act_mul`."""
        self.act_mul(gate_up, out, block, "silu")

    def act_mul(self, gate_up, out, block=0, activation="silu", limit=None):
        """out = act(gate) * up, act one of `ACTIVATIONS`.  `block` 0: a row of gate_up is all gate columns,
        then all up columns; b > 0: runs of b gate columns, each followed by the b up columns of the same features.
        `clamped_swish` with `limit` L is min(g, L) * sigmoid(1.702 min(g, L)) * (clamp(u, -L, L) + 1)."""
        _dense(gate_up, self.dtype, "gate_up")
        _dense(out, self.dtype, "activation")
        n, inter = out.shape
        self.launches += 1
        _check(self.core.shrike_act_mul_limit(_ptr(gate_up), _ptr(out), self.code, n, inter, block,
                                              self.ACTIVATIONS[activation], self._limit(activation, limit), self._stream()),
               "act_mul")

    @staticmethod
    def _limit(activation, limit) -> float:
        if activation == "clamped_swish":
            if limit is None or not limit > 0:
                raise KernelError("the clamped activation needs a positive limit")
            return float(limit)
        return 0.0

    @property
    def gated_rows(self) -> int:
        """How a gated feed-forward should interleave the rows of its fused gate/up matrix for
        `linear_gated`: runs of this many gate rows, each followed by the up rows of the same
        features.  0: keep gate rows, then up rows (no fused activation in this mode)."""
        return 16 if self.dtype == torch.bfloat16 and self.gemm_tc is not None else 0

    def linear_gated(self, x, w, out, activation="silu", limit=None) -> bool:
        """act(x Wg^T) * (x Wu^T) into `out` [N, I] in one kernel, for `w` [2 I, K] interleaved as
        `gated_rows` says.  Returns False when this shape is not served (many tokens: the caller
        then runs the product and the activation kernel, the latter with block=gated_rows)."""
        n, k = x.shape
        rows = w.shape[0]
        if (self.gated_rows == 0 or n > self.tensor_core_gemm_max_tokens or k % 8 or rows % 32
                or tuple(out.shape) != (n, rows // 2) or w.shape[1] != k):
            return False
        _dense(x, torch.bfloat16, "linear input")
        _dense(w, torch.bfloat16, "linear weight")
        _dense(out, torch.bfloat16, "activation")
        self.launches += 1
        _check(self.gemm_tc.shrike_gemm_tc_gated_act_limit(_ptr(x), _ptr(w), _ptr(out), n, rows, k,
                                                           self.ACTIVATIONS[activation], self._limit(activation, limit),
                                                           _ptr(self.status), self._stream()),
               "gemm_tcgen05")
        return True

    def tanh_norm(self, resid, terms=(), row_add=None, rows=None, norms=()):
        """resid += sum over `terms` of scale * pending (each `(tensor, scale)`, the tensor float32 [N, W] or
        a K-split stack [P, N, W]) + `row_add` (float32 [W], added to every row); then, for each of up to two
        `norms` `(alpha, weight, bias, out)`, out = tanh(alpha x) * weight + bias of the summed row.  With
        `rows` (int32 [R]) only `out[r]` for row rows[r] is written, the residual stays."""
        _dense(resid, torch.float32, "residual")
        n, width = resid.shape
        if len(terms) > 4 or len(norms) > 2:
            raise KernelError("tanh_norm takes at most four pending sums and two norms")
        count = rows.shape[0] if rows is not None else n
        data = (_P * 4)()
        partials, strides, scales = (_I * 4)(), (_LL * 4)(), (_F * 4)()
        for index, (tensor, scale) in enumerate(terms):
            _dense(tensor, torch.float32, "pending sum")
            if tuple(tensor.shape[-2:]) != (n, width):
                raise KernelError(f"pending sum {tuple(tensor.shape)} does not fit the residual {tuple(resid.shape)}")
            data[index] = tensor.data_ptr()
            partials[index], strides[index] = self._stack(tensor)
            scales[index] = float(scale)
        alpha, weight, bias, out = (_F * 2)(), (_P * 2)(), (_P * 2)(), (_P * 2)()
        out_code = 0
        for index, (a, w, b, o) in enumerate(norms):
            _dense(w, torch.float32, "norm weight")
            _dense(b, torch.float32, "norm bias")
            if tuple(o.shape) != (count, width) or not o.is_contiguous():
                raise KernelError(f"norm output {tuple(o.shape)} does not fit {count} rows of {width}")
            alpha[index], weight[index], bias[index], out[index] = float(a), w.data_ptr(), b.data_ptr(), o.data_ptr()
            out_code = _DTYPE_CODE[o.dtype]
        if rows is not None:
            _dense(rows, torch.int32, "rows")
        self.launches += 1
        _check(self.core.shrike_tanh_norm(_ptr(resid), data, partials, strides, scales, len(terms), _ptr(row_add), _ptr(rows),
                                          len(norms), alpha, weight, bias, out, out_code, count, width, self._stream()),
               "tanh_norm")

    def head_prep(self, fused, bias, positions, inv_freq, rot, q_weight, k_weight, eps, q_out, keys, values, slots,
                  gate_out, num_heads, num_kv_heads, dim, vdim, padded, whole_norm=False, value_norm=False):
        """A fused q|k|v(|gate) projection ([N, total] float32 or a K-split stack) made ready for paged
        attention: `bias` ([total] or None) added; q and k divided by their root mean square per head and
        scaled by `q_weight` / `k_weight` ([dim], None: left as they are); the first `rot` dimensions of
        every q and k head rotated, dimension i with i + rot/2, by position * inv_freq[i]; q to `q_out`
        [N, H * padded], k and v into their pages, heads `padded` elements apart (padding zeroed); with
        `gate_out` (float32 [N, H]) the sigmoid of the last H columns.  `whole_norm`: q and k are divided by the
        root mean square of their whole projections instead (all heads at once), `q_weight` [H dim] and `k_weight`
        [G dim] one number a column.  `value_norm`: every value head over its own root mean square.  `num_kv_heads`
        0: the projection holds queries alone."""
        _dense(fused, torch.float32, "fused projection")
        _dense(q_out, self.dtype, "q")
        partials, stride = self._stack(fused)
        num_slots = 0
        if keys is not None:
            _dense(keys, self.dtype, "key cache")
            _dense(values, self.dtype, "value cache")
            num_slots = keys.shape[0] * keys.shape[1]
        self.launches += 1
        _check(self.core.shrike_head_prep_norms(
            _ptr(fused), partials, stride, fused.shape[-1], _ptr(bias), _ptr(positions), _ptr(inv_freq), rot if inv_freq is not None else 0,
            _ptr(q_weight), _ptr(k_weight), eps, _ptr(q_out), _ptr(keys), _ptr(values), _ptr(slots), _ptr(gate_out),
            self.code, fused.shape[-2], num_heads, num_kv_heads, dim, vdim, padded, num_slots, int(bool(whole_norm)),
            int(bool(value_norm)), self._stream()), "head_prep")

    def matrix_memory(self, fused, gate_bias, state, q_start, state_slot, numerator, denominator, weight, eps, out,
                      num_seqs, num_heads, dim, vdim, cap, floor, longest=0):
        """The matrix-memory recurrence over the batch's new tokens and its gated, normed output.  `longest`: the
        most new tokens a sequence of the batch brings (the batch's shape, known on the host); long portions run
        as products over 64 tokens at a time, short ones and single tokens as a walk, with the same result.

        `fused` ([N, total] float32 or a K-split stack): q (H dim) | k (H dim) | v (H vdim) | output gate
        (H vdim) | input gate (H) | forget gate (H); `gate_bias` float32 [2 H].  `state` float32
        [slots, H, at least dim * vdim + dim + 1] (S, z, m of every head; a multiple of four floats keeps the heads
        on 16-byte borders) is read and left updated for the slots
        `state_slot` names (-1: the sequence is skipped).  `out` [N, H * vdim]: each head's o over its root
        mean square, times `weight`, times the sigmoid of the output gate."""
        _dense(fused, torch.float32, "fused projection")
        _dense(state, torch.float32, "state")
        _dense(out, self.dtype, "mixer output")
        partials, stride = self._stack(fused)
        total, n = fused.shape[-1], fused.shape[-2]
        if state.dim() != 3 or state.shape[1] != num_heads or state.shape[2] < dim * vdim + dim + 1:
            raise KernelError(f"state {tuple(state.shape)} does not fit {num_heads} heads of {dim} x {vdim}")
        chunk_state = chunk_info = token_info = chunk_scores = None
        if longest >= 16:   # long portions: products over chunks of 64 tokens, which hand each other scratch
            chunks = self.core.shrike_matrix_memory_chunks(n, num_seqs)
            sizes = (chunks * num_heads * (dim * vdim + dim), chunks * num_heads * 4, n * num_heads * 4, chunks * num_heads * 4096)
            held = self._memory_scratch
            if held is None or any(t.numel() < size for t, size in zip(held, sizes)):
                held = tuple(torch.empty(max(2 * size, 1024), dtype=torch.float32, device=self.device) for size in sizes)
                self._memory_scratch = held
                self.generation += 1
            chunk_state, chunk_info, token_info, chunk_scores = held
        self.launches += 5 if chunk_state is not None else 2
        _check(self.core.shrike_matrix_memory_scan(
            _ptr(fused), partials, stride, total, _ptr(gate_bias), _ptr(state), _ptr(q_start), _ptr(state_slot),
            _ptr(numerator), _ptr(denominator), num_seqs, num_heads, dim, vdim, state.shape[0], cap, float(dim) ** -0.5, floor,
            int(longest), state.shape[2], n, _ptr(chunk_state), _ptr(chunk_info), _ptr(token_info), _ptr(chunk_scores),
            self._stream()),
            "matrix_memory_scan")
        _check(self.core.shrike_matrix_memory_out(
            _ptr(numerator), _ptr(denominator), _ptr(fused), partials, stride, total, 2 * num_heads * dim + num_heads * vdim,
            _ptr(weight), eps, _ptr(out), self.code, n, num_heads, vdim, self._stream()), "matrix_memory_out")

    DECAY_CHUNK_FROM = 32   # a sequence that brings at least this many tokens runs its decayed scan over runs of tokens

    def decay_scan(self, fused, decays, state, q_start, state_slot, out, num_seqs, num_heads, dim, vdim, longest=0):
        """Linear attention with a decay per head over the batch's new tokens: S <- decays[h] S + k v^T, o = S^T q, with
        q (H dim) | k (H dim) | v (H vdim) the SiLU of the first columns of `fused` ([N, total] float32 or a K-split
        stack).  `state` float32 [slots, H, at least dim * vdim] is read and left updated for the slots `state_slot`
        names (-1: the sequence is skipped); `out` float32 [N, H * vdim].  `longest`: the most new tokens a sequence
        of the batch brings (the batch's shape, known on the host); long portions run as products over 64 tokens at a
        time, short ones and single tokens as a walk, with the same result up to the order of the sums."""
        _dense(fused, torch.float32, "fused projection")
        _dense(state, torch.float32, "state")
        _dense(out, torch.float32, "scan output")
        _dense(decays, torch.float32, "decays")
        partials, stride = self._stack(fused)
        total, n = fused.shape[-1], fused.shape[-2]
        if state.dim() != 3 or state.shape[1] != num_heads or state.shape[2] < dim * vdim or decays.numel() != num_heads:
            raise KernelError(f"state {tuple(state.shape)} does not fit {num_heads} heads of {dim} x {vdim}")
        chunk_state = None
        if longest >= self.DECAY_CHUNK_FROM:
            need = self.core.shrike_decay_scan_chunks(n, num_seqs) * num_heads * dim * vdim
            held = self._decay_scratch
            if held is None or held.numel() < need:
                held = torch.empty(max(2 * need, 1024), dtype=torch.float32, device=self.device)
                self._decay_scratch = held
                self.generation += 1
            chunk_state = held
        self.launches += 4 if chunk_state is not None else 1
        _check(self.core.shrike_decay_scan(
            _ptr(fused), partials, stride, total, _ptr(decays), _ptr(state), _ptr(q_start), _ptr(state_slot), _ptr(out),
            num_seqs, num_heads, dim, vdim, state.shape[0], state.shape[2], int(longest), self.DECAY_CHUNK_FROM, n,
            _ptr(chunk_state), self._stream()), "decay_scan")

    def norm_gate(self, x, gate_source, gate_at, weight, eps, out):
        """out = x (float32 [N, W]), each row over its root mean square times `weight` (float32 [W]; None: the row as it
        is), times the sigmoid of columns `gate_at` .. `gate_at` + W of `gate_source` ([N, total] float32 or a K-split
        stack; None: no gate), in the type of `out`."""
        _dense(x, torch.float32, "rows")
        _dense(out, self.dtype, "gated rows")
        n, width = x.shape
        partials, stride, row_width = 1, 0, 0
        if gate_source is not None:
            _dense(gate_source, torch.float32, "fused projection")
            partials, stride = self._stack(gate_source)
            row_width = gate_source.shape[-1]
            if gate_at + width > row_width:
                raise KernelError("the gate's columns lie outside the fused projection")
        self.launches += 1
        _check(self.core.shrike_norm_gate(_ptr(x), _ptr(gate_source), partials, stride, row_width, gate_at, _ptr(weight), eps,
                                          _ptr(out), self.code, n, width, self._stream()), "norm_gate")

    def latent_rope_store(self, fused, latent_weight, eps, positions, inv_freq, gain, q_out, latents, slots, heads, rank,
                          rot, padded):
        """A fused projection ([N, total] float32 or a K-split stack) whose row is `heads` x [rank | rot] queries and then
        [rank | rot] of the token itself, made ready for attention over a cached latent: every [rot] part rotated,
        dimension i with i + rot/2, by position * inv_freq[i] with cos and sin times `gain`; the token's [rank] part
        divided by its root mean square and scaled by `latent_weight`.  Queries go to `q_out` [N, heads * padded], the
        token's [rank | rot] into its page row (`latents`, rows of `padded`; None: not stored); padding is zeroed."""
        _dense(fused, torch.float32, "fused projection")
        _dense(q_out, self.dtype, "q")
        partials, stride = self._stack(fused)
        num_slots = 0
        if latents is not None:
            _dense(latents, self.dtype, "latent cache")
            num_slots = latents.shape[0] * latents.shape[1]
        self.launches += 1
        _check(self.core.shrike_latent_rope_store(
            _ptr(fused), partials, stride, fused.shape[-1], _ptr(latent_weight), eps, _ptr(positions), _ptr(inv_freq),
            float(gain), _ptr(q_out), _ptr(latents), _ptr(slots), self.code, fused.shape[-2], heads, rank, rot, padded,
            num_slots, self._stream()), "latent_rope_store")

    def concat_cast(self, resid, terms, other, out):
        """resid (float32 [N, W]) += the pending `terms` ((tensor, scale), each float32 [N, W] or a K-split stack); then
        out[N, 2 W] = [resid | other] in the type of `out` (`other` float32 [N, W])."""
        _dense(resid, torch.float32, "residual")
        _dense(other, torch.float32, "second half")
        _dense(out, self.dtype, "joined rows")
        terms = list(terms)
        n, width = resid.shape
        while len(terms) > 4:   # more pending sums than one launch adds: the first ones go into the residual alone
            self.tanh_norm(resid, terms[:4])
            terms = terms[4:]
        count = len(terms)
        data, parts = (ctypes.c_void_p * 4)(), (ctypes.c_int * 4)()
        strides, scales = (ctypes.c_longlong * 4)(), (ctypes.c_float * 4)()
        for index, (tensor, scale) in enumerate(terms):
            _dense(tensor, torch.float32, "pending sum")
            data[index] = tensor.data_ptr()
            parts[index], strides[index] = self._stack(tensor)
            scales[index] = float(scale)
        self.launches += 1
        _check(self.core.shrike_concat_cast(_ptr(resid), data, parts, strides, scales, count, _ptr(other), _ptr(out), self.code,
                                            n, width, self._stream()), "concat_cast")

    def head_linear(self, x, w, out, heads):
        """out[n, h, :] = w[h] x[n, h, :]: x [N, heads * P] in the engine's type, w [heads, V, P], out float32
        [N, heads * V].  One batched library product over the heads, reading and writing in place through strides."""
        n = x.shape[0]
        _dense(x, self.dtype, "head inputs")
        _dense(out, torch.float32, "head outputs")
        if w.dim() != 3 or w.shape[0] != heads or x.shape[1] != heads * w.shape[2] or out.shape[1] != heads * w.shape[1]:
            raise KernelError(f"head_linear: x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
        self.library_calls += 1
        a = x.view(n, heads, w.shape[2]).transpose(0, 1)          # [heads, N, P]
        target = out.view(n, heads, w.shape[1]).transpose(0, 1)   # [heads, N, V]
        if self.dtype == torch.float32:
            torch.bmm(a, w.transpose(1, 2), out=target)
        else:
            torch.bmm(a, w.transpose(1, 2), out_dtype=torch.float32, out=target)

    def route_top(self, x, router, shared_gate, weights, top, renorm_eps, scoring="softmax", renormalise=True):
        """weights [N, E (+ 1)] float32: softmax(router x) over all E experts in 32-bit, the `top` largest
        divided by their sum (+ renorm_eps), 0 elsewhere; a last column, when there is one, holds
        sigmoid(shared_gate . x) (1 when `shared_gate` is None).  `scoring` "sigmoid": an expert's score is the
        sigmoid of its own logit; `renormalise` False: the chosen keep their scores as they are."""
        _dense(x, self.dtype, "router input")
        _dense(router, torch.float32, "router weight")
        _dense(weights, torch.float32, "expert weights")
        self.launches += 1
        _check(self.core.shrike_route_top_scores(_ptr(x), self.code, _ptr(router), _ptr(shared_gate), _ptr(weights), x.shape[0],
                                                 x.shape[1], router.shape[0], top, weights.shape[1], renorm_eps,
                                                 int(scoring == "sigmoid"), int(bool(renormalise)), self._stream()), "route_top")

    def act_mul_blocks(self, gate_up, weights, out, experts, each, activation="silu", limit=None, weight_on="output"):
        """out[n, c] = act(gate[n, c]) * up[n, c] * weights[n, e(c)] for gate_up [N, 2 I] (gate columns, then up
        columns): column c belongs to expert c // each while c < experts * each, else to the shared expert
        (the last column of `weights`).  `weight_on` "input": the weight w multiplies the expert's input, which
        reaches gate and up alike, out = act(w gate) * (w up)."""
        _dense(gate_up, self.dtype, "gate_up")
        _dense(out, self.dtype, "activation")
        _dense(weights, torch.float32, "expert weights")
        n, inter = out.shape
        self.launches += 1
        _check(self.core.shrike_act_mul_blocks_at(_ptr(gate_up), _ptr(weights), _ptr(out), self.code, n, inter, experts, each,
                                                  weights.shape[1], self.ACTIVATIONS[activation], self._limit(activation, limit),
                                                  int(weight_on == "input"), self._stream()), "act_mul_blocks")

    # ---- several residual streams, a short convolution, a gated recurrence -----------------------------
    def stream_norm(self, streams, pending, join, in_weights, norm_weight, eps, out, rows=None, sum_out=None):
        """`streams` float32 [N, S, W].  `pending` (a list of (tensor, scale), each tensor float32 [N, W] or a K-split
        stack) with `join` = (mix [S, S] indexed (from, to), out [S], layer scale [W] or None): the sublayer result
        y = layer scale * sum of the pending terms joins the streams, x_t <- sum_s mix[s, t] x_s + out[t] y (`join`
        None: nothing is pending).  Then u = sum_t in_weights[t] x_t (`in_weights` None: the plain sum) and
        out = u / sqrt(mean(u^2) + eps) * norm_weight.  With `rows` (int32 [R]) only those tokens are read, the
        streams stay as they are and out is [R, W].  `sum_out` (float32, the shape of out) receives u itself."""
        _dense(streams, torch.float32, "residual streams")
        n, count, width = streams.shape
        terms = list(pending or []) if join is not None else []
        if len(terms) > 4:
            raise KernelError("stream_norm takes at most four pending sums")
        data, partials, strides, scales = (_P * 4)(), (_I * 4)(), (_LL * 4)(), (_F * 4)()
        for index, (tensor, scale) in enumerate(terms):
            _dense(tensor, torch.float32, "pending sum")
            if tuple(tensor.shape[-2:]) != (n, width):
                raise KernelError(f"pending sum {tuple(tensor.shape)} does not fit {n} rows of {width}")
            data[index] = tensor.data_ptr()
            partials[index], strides[index] = self._stack(tensor)
            scales[index] = float(scale)
        mix, out_w, layer_scale = join if join is not None else (None, None, None)
        for name, tensor in (("mix", mix), ("out", out_w), ("layer scale", layer_scale), ("in", in_weights), ("norm weight", norm_weight)):
            if tensor is not None:
                _dense(tensor, torch.float32, name)
        count_rows = rows.shape[0] if rows is not None else n
        if rows is not None:
            _dense(rows, torch.int32, "rows")
        for tensor in (out, sum_out):
            if tensor is not None and (tuple(tensor.shape) != (count_rows, width) or not tensor.is_contiguous()):
                raise KernelError(f"stream_norm output {tuple(tensor.shape)} does not fit {count_rows} rows of {width}")
        self.launches += 1
        _check(self.core.shrike_stream_norm(
            _ptr(streams), data, partials, strides, scales, len(terms), _ptr(mix), _ptr(out_w), _ptr(layer_scale),
            _ptr(in_weights), _ptr(norm_weight), eps, _ptr(out), -1 if out is None else _DTYPE_CODE[out.dtype], _ptr(sum_out),
            _ptr(rows), count_rows, width, count, self._stream()), "stream_norm")

    def short_conv(self, fused, bias, taps, state, q_start, state_slot, seq_of_token, out, num_seqs, channels):
        """out[t, c] = sum_j taps[c, j] u[t - T + 1 + j, c] for the first `channels` columns of the projection
        u = `fused` (+ `bias`) ([N, total] float32 or a K-split stack), the other columns copied; the T - 1 values
        before a portion's first token come from `state` float32 [slots, T - 1, channels] (zeros when the request
        was just opened), which is left holding the portion's last T - 1 projected values."""
        _dense(fused, torch.float32, "fused projection")
        _dense(taps, torch.float32, "convolution taps")
        _dense(out, torch.float32, "convolved projection")
        _dense(state, torch.float32, "convolution state")
        partials, stride = self._stack(fused)
        n, total = fused.shape[-2], fused.shape[-1]
        if tuple(taps.shape)[0] != channels or tuple(state.shape[1:]) != (taps.shape[1] - 1, channels) or tuple(out.shape) != (n, total):
            raise KernelError("short_conv: taps [channels, T], state [slots, T - 1, channels], out [N, total]")
        self.launches += 2 if taps.shape[1] > 1 else 1
        _check(self.core.shrike_short_conv(_ptr(fused), partials, stride, total, _ptr(bias), _ptr(taps), _ptr(state), _ptr(q_start),
                                           _ptr(state_slot), _ptr(seq_of_token), _ptr(out), n, channels, taps.shape[1], num_seqs,
                                           state.shape[0], self._stream()), "short_conv")

    GATED_SCAN_RUN = 64       # tokens of a run when a portion is cut into runs that walk side by side
    GATED_SCAN_RUNS_FROM = 192   # the longest portion of a batch from which on that is done

    def gated_scan(self, fused, f_bias, lower, state, q_start, state_slot, out, num_seqs, num_heads, dim, vdim, q_lens=None):
        """The gated linear recurrence over the batch's new tokens: per head S <- diag(f) S + (1 - f) v^T, o = S^T q,
        with q = silu(.), f = lower + (1 - lower) sigmoid(. + f_bias) and v the columns q (H dim) | f (H dim) | v (H vdim)
        of `fused` ([N, total] float32 or a K-split stack).  `state` float32 [slots, H, at least dim * vdim] is read
        and left updated for the slots `state_slot` names (-1: zeros out, nothing kept); `out` float32 [N, H * vdim].
        `q_lens` (the batch's lengths, host): long portions are cut into runs of tokens that walk side by side."""
        _dense(fused, torch.float32, "fused projection")
        _dense(state, torch.float32, "recurrence state")
        _dense(out, torch.float32, "recurrence output")
        partials, stride = self._stack(fused)
        run, runs, run_state, run_decay, run_first = 0, 0, None, None, None
        if q_lens is not None and max(q_lens) >= self.GATED_SCAN_RUNS_FROM:
            run = self.GATED_SCAN_RUN
            runs = sum(-(-length // run) for length in q_lens)
            need = runs * num_heads * (dim * vdim + dim) + num_seqs + 1
            if self._scan_scratch is None or self._scan_scratch.numel() < need:
                self._scan_scratch = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=self.device)
                self.generation += 1
            scratch = self._scan_scratch
            run_state = scratch[: runs * num_heads * dim * vdim]
            run_decay = scratch[runs * num_heads * dim * vdim: runs * num_heads * (dim * vdim + dim)]
            run_first = scratch[runs * num_heads * (dim * vdim + dim): need].view(torch.int32)
        self.launches += 4 if run else 1
        _check(self.core.shrike_gated_scan(
            _ptr(fused), partials, stride, fused.shape[-1], _ptr(f_bias), _ptr(lower), _ptr(state), _ptr(q_start), _ptr(state_slot),
            _ptr(out), num_seqs, num_heads, dim, vdim, state.shape[-1], state.shape[0], run, _ptr(run_state), _ptr(run_decay),
            _ptr(run_first), runs, int(self.dtype == torch.bfloat16), self._stream()), "gated_scan")

    def head_rms(self, x, weight, eps, out, heads):
        """out[n, h, :] = x[n, h, :] / sqrt(mean(x[n, h, :]^2) + eps) * weight for x float32 [N, heads * size]."""
        _dense(x, torch.float32, "head outputs")
        n, width = x.shape
        self.launches += 1
        _check(self.core.shrike_head_rms(_ptr(x), _ptr(weight), _ptr(out), _DTYPE_CODE[out.dtype], n, heads, width // heads, eps,
                                         self._stream()), "head_rms")

    def sample(self, logits, temperature, top_p, seeds, out):
        _dense(logits, torch.float32, "logits")
        _dense(temperature, torch.float32, "temperature")
        _dense(top_p, torch.float32, "top_p")
        _dense(seeds, torch.int64, "seeds")
        _dense(out, torch.int32, "sampled tokens")
        rows, vocab = logits.shape
        need = max(rows, 64) * self.core.shrike_sample_slices(vocab)
        if self._sample_scratch is None or self._sample_scratch[0].numel() < need:
            self._sample_scratch = (torch.empty(2 * need, dtype=torch.float32, device=self.device),
                                    torch.empty(2 * need, dtype=torch.int32, device=self.device))
            self.generation += 1
        values, indices = self._sample_scratch
        self.launches += 2
        _check(self.core.shrike_sample(_ptr(logits), _ptr(temperature), _ptr(top_p), _ptr(seeds), _ptr(out),
                                       _ptr(values), _ptr(indices), rows, vocab, _ptr(self.status), self._stream()),
               "sample")
