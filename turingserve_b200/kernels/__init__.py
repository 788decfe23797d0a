"""The CUDA kernels (sm_100a) behind one object, ``ops()``.

The library is built in-tree at the first call (``kernels.build``) and loaded with ctypes; every
function takes raw device pointers and the current CUDA stream.  There is no other backend: on a
machine without the library and without nvcc, or without a CUDA device, ``ops()`` raises.

Kernels and their reference counterparts (turingserve/ops/__init__.py:15-19 lists the op
namespace): embedding, rmsnorm (+residual), linear, rope fused with the cache write, paged
attention, silu*mul, sampling.  bfloat16 matrix products go to cuBLAS through ``torch.mm`` where
the reference uses ``F.linear`` (turingserve/ops/triton_ops.py:74-76), unless a hand-written
tensor-core kernel takes the shape; float32 products always use this library's FFMA kernel.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch

from turingserve_b200.kernels.build import build, library_path

_OPS = None

c_int, c_float, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16, not {dtype}") from None


class KernelError(RuntimeError):
    pass


class Deferred:
    """A product whose split-K partial sums still sit in scratch ([splits, M, N] float32): the norm
    that consumes it finishes the sum in its own kernel.  Quacks like a tensor as far as shape,
    dtype and device go; anything else must call ``ops().materialize`` first."""

    def __init__(self, part: torch.Tensor, splits: int, shape, dtype, bias, out: torch.Tensor) -> None:
        self.part, self.splits, self.shape, self.dtype, self.bias = part, splits, tuple(shape), dtype, bias
        self.device = part.device
        self.out = out                      # the buffer the finished product belongs in


class LazyProduct:
    """A few-token product that has not been launched yet: out = x @ w^T + bias.  The norm that gets it
    together with a residual launches it as ONE kernel that also sums its K splits (a thread-block
    cluster) and adds the result to the residual in place; any other consumer has it launched the
    ordinary way (``ops().materialize``, or as a ``Deferred``).  Shape, dtype and device as a tensor's."""

    def __init__(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, bias) -> None:
        self.out, self.x, self.w, self.bias = out, x, w, bias
        self.shape, self.dtype, self.device = tuple(out.shape), out.dtype, out.device


class CudaOps:
    """ctypes front of ``libturingserve_b200.so``."""

    ABI = 14
    UNSUPPORTED = -4            # a kernel's refusal of a shape or layout another kernel takes

    def __init__(self, lib_path: str) -> None:
        self.lib_path = lib_path
        self.lib = ctypes.CDLL(lib_path)
        self.lib.ts_last_error.restype = ctypes.c_char_p
        if self.lib.ts_abi_version() != self.ABI:
            raise KernelError(f"{lib_path} has ABI {self.lib.ts_abi_version()}, this package needs {self.ABI}")
        P, I, F = c_void_p, c_int, c_float
        sigs = {
            "ts_embedding": [P, P, P, I, I, I, I, P],
            "ts_gather_rows": [P, P, P, I, I, I, P],
            "ts_rmsnorm": [P, P, P, P, F, I, I, I, I, P],
            "ts_silu_mul": [P, P, I, I, I, P],
            "ts_silu_mul_ex": [P, P, I, I, I, I, P],
            "ts_linear_tc_gated": [P, P, P, I, I, I, P],
            "ts_linear_tc_resid": [P, P, P, P, I, I, I, I, P],
            "ts_linear_pair": [P, P, P, P, I, I, I, I, P],
            "ts_linear_pair_qkv": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
            "ts_linear_tc_qkv_rope": [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
            "ts_rope_kv_write": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
            "ts_rope_kv_write_ex": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, P, I, P, P],
            "ts_attention_generic": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P],
            "ts_linear_simt": [P, P, P, P, P, I, I, I, I, I, P],
            "ts_attention_decode": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P],
            "ts_attention_decode_tma": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P],
            "ts_attention_prefill": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P],
            "ts_attention_prefill_tc": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P],
            "ts_linear_tc": [P, P, P, P, P, I, I, I, I, I, P],
            "ts_linear_tc_ex": [P, P, P, P, P, I, I, I, I, I, I, P, P],
            "ts_reduce_rmsnorm": [P, P, I, P, P, P, F, I, I, I, P],
            "ts_feed_tokens": [P, P, P, P, I, I, P],
            "ts_sample": [P, P, P, P, I, I, P, P],
            "ts_penalize": [P, P, P, P, I, I, P],
            "ts_sample_greedy": [P, P, I, I, P, P, P, P],
            "ts_clear_status": [P],
            "ts_decode_step": [P, I, I, P],
            "ts_decode_step_encode_map": [P, P, I, I],
            "ts_poke_status": [I, I, P],
            "ts_rmsnorm_wide": [P, P, P, P, P, F, I, I, I, I, I, P, I, P, F, P, P, P],
            "ts_activation_parts": [P, P, I, P, I, I, I, I, P],
            "ts_gated_rmsnorm": [P, P, P, I, P, F, I, I, I, I, P],
            "ts_activation": [P, P, ctypes.c_longlong, I, I, P],
            "ts_lightning": [P, P, I, P, P, P, P, I, I, I, I, I, P],
            "ts_kv_write_pair": [P, I, I, I, P, P, P, I, I, I, I, I, I, P],
            "ts_attention_diff": [P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, F, F, F, F, I, P],
            "ts_attention_diff_mma": [P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, F, F, F, F, P, P, I, I, P],
            "ts_router_topk": [P, P, P, P, I, I, I, I, I, I, I, P, P],
            "ts_moe_align": [P, I, I, P, P, P, P, I, P],
            "ts_grouped_linear": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P],
            "ts_moe_combine": [P, P, P, P, I, I, I, I, P, P, P, P],
            "ts_hyper_norm": [P, P, P, P, I, P, P, P, P, P, F, I, I, I, I, F, I, P],
            "ts_ssm_prepare": [P, P, I, I, I, P, P, P, P, P, ctypes.c_longlong, ctypes.c_longlong, P, P, P, I, I, I, I, I, P],
            "ts_ssm_scan": [P, P, P, I, I, P, ctypes.c_longlong, P, P, P, I, I, I, I, I, I, I, I, P],
            "ts_lightning_ex": [P, P, I, P, P, P, P, I, I, I, I, I, I, P],
            "ts_gated_group_rmsnorm": [P, I, P, P, I, P, F, I, I, I, I, I, F, I, P],
            "ts_gate_mul": [P, I, P, I, P, I, I, I, I, F, I, P],
            "ts_act_mul": [P, P, I, I, I, I, I, P],
            "ts_rope_pairs_write": [P, I, I, I, P, P, F, I, P, P, P, I, I, I, I, I, I, I, P],
            "ts_moe_gather": [P, P, P, P, I, I, I, I, P],
            "ts_delta_prepare": [P, P, I, P, P, P, P, ctypes.c_longlong, P, P, P, I, I, I, I, I, I, F, I, P],
            "ts_delta_scan": [P, P, P, I, P, ctypes.c_longlong, P, P, I, I, I, I, I, I, I, I, P],
            "ts_head_gated_rmsnorm": [P, P, P, I, P, F, I, I, I, I, P],
            "ts_attention_biased": [P, I, I, P, I, I, P, P, P, P, P, I, I, I, I, I, I, I, I, F, F, P, I, I, P, P, I, I, P, P],
            "ts_attention_biased_mma": [P, I, I, P, I, I, P, P, P, P, P, I, I, I, I, I, I, I, I, F, F, P, I, I, P, P, I, I, P, P],
            "ts_rope_headnorm_write": [P, I, I, I, P, P, I, I, F, P, P, P, I, I, I, I, I, I, I, P, I, P],
            "ts_rope_headnorm_write_supports_parts": [I, I, I, I],
            "ts_rms_rows": [P, P, I, I, I, P, F, I, I, P],
            "ts_qk_rownorm_write": [P, I, P, P, F, P, F, I, P, P, P, I, I, I, I, I, I, P],
            "ts_latent_kv_write": [P, I, I, P, F, P, P, F, I, P, P, I, I, I, I, I, P],
            "ts_rotate_pairs": [P, I, I, P, I, I, P, P, F, I, I, I, I, I, P],
            "ts_batched_linear": [P, I, I, P, I, I, P, I, I, I, I, I, P],
        }
        for name, args in sigs.items():
            fn = getattr(self.lib, name)
            fn.argtypes = args
            fn.restype = c_int
        self.lib.ts_attention_diff_mma_supported.argtypes = [I, I, I, I, I]
        self.lib.ts_attention_diff_mma_supported.restype = c_int
        self.lib.ts_attention_diff_mma_scratch_floats.argtypes = [I, I, I, I]
        self.lib.ts_attention_diff_mma_scratch_floats.restype = ctypes.c_longlong
        self.lib.ts_set_delta_rows.argtypes = [I]
        self.lib.ts_set_delta_rows.restype = None
        self.lib.ts_set_delta_rows(int(os.environ.get("TURINGSERVE_B200_DELTA_ROWS", "0")))
        self.lib.ts_attention_biased_mma_supported.argtypes = [I, I, I, I, I, I]
        self.lib.ts_attention_biased_mma_supported.restype = c_int
        self.lib.ts_attention_biased_mma_chunk.argtypes = [I, I, I]
        self.lib.ts_attention_biased_mma_chunk.restype = c_int
        self.lib.ts_attention_biased_mma_scratch_floats.argtypes = [I, I, I, I, I, I]
        self.lib.ts_attention_biased_mma_scratch_floats.restype = ctypes.c_longlong
        self.lib.ts_attention_biased_scratch_floats.argtypes = [I, I, I, I, I, I]
        self.lib.ts_attention_biased_scratch_floats.restype = ctypes.c_longlong
        self.lib.ts_rmsnorm_wide_takes_parts.argtypes = [I]
        self.lib.ts_rmsnorm_wide_takes_parts.restype = c_int
        self.lib.ts_moe_tile_rows.argtypes = []
        self.lib.ts_moe_tile_rows.restype = c_int
        self.lib.ts_attention_decode_supported.argtypes = [I, I, I, I]
        self.lib.ts_attention_decode_supported.restype = c_int
        self.lib.ts_attention_decode_tma_supported.argtypes = [I, I, I, I, I]
        self.lib.ts_attention_decode_tma_supported.restype = c_int
        self.lib.ts_attention_decode_tma_status.argtypes = []
        self.lib.ts_attention_decode_tma_status.restype = c_int
        self.lib.ts_attention_decode_tma_blocks_per_sm.argtypes = [I, I]
        self.lib.ts_attention_decode_tma_blocks_per_sm.restype = c_int
        # decode attention: "tma" the kernel built for streaming many keys (pages of a multiple of 16
        # tokens), "cp" the one built for the shortest chain, "auto" by the step's streaming_decode
        self.decode_kernel = os.environ.get("TURINGSERVE_B200_DECODE_ATTENTION", "auto")
        self.decode_stages = int(os.environ.get("TURINGSERVE_B200_DECODE_STAGES", "3"))
        self.lib.ts_set_decode_tma_cluster_max.argtypes = [I]
        self.lib.ts_set_decode_tma_cluster_max.restype = None
        if "TURINGSERVE_B200_DECODE_TMA_CLUSTER" in os.environ:
            self.lib.ts_set_decode_tma_cluster_max(int(os.environ["TURINGSERVE_B200_DECODE_TMA_CLUSTER"]))
        # the "cp" kernel where the rule asks for 16 splits: 8 splits of 8 warps instead.  2: whenever those
        # blocks fit one per SM (merged as clusters where all clusters fit the chip, else by the ticket);
        # 1: only as clusters; 0: never
        self.lib.ts_set_pair_tile_width.argtypes = [I]
        self.lib.ts_set_pair_tile_width.restype = None
        self.lib.ts_set_decode_wide.argtypes = [I]
        self.lib.ts_set_decode_wide.restype = None
        self.lib.ts_set_decode_wide(int(os.environ.get("TURINGSERVE_B200_DECODE_WIDE", "2")))
        self.lib.ts_linear_tc_qkv_rope_scratch_floats.argtypes = [I, I, I]
        self.lib.ts_linear_tc_qkv_rope_scratch_floats.restype = ctypes.c_longlong
        self.lib.ts_sample_greedy_parts.argtypes = [I]
        self.lib.ts_sample_greedy_parts.restype = c_int
        self.lib.ts_rope_kv_write_fused_supported.argtypes = [I, I, I]
        self.lib.ts_rope_kv_write_fused_supported.restype = c_int
        self.lib.ts_linear_tc_supported.argtypes = [I, I, I]
        self.lib.ts_linear_tc_supported.restype = c_int
        self.lib.ts_linear_tc_status.argtypes = []
        self.lib.ts_linear_tc_status.restype = c_int
        # which bfloat16 products run on this library's tcgen05 kernel: "tc" all of them, "auto" those
        # with at most 128 rows (decode), "library" none (cuBLAS through torch.mm)
        self.gemm_mode = os.environ.get("TURINGSERVE_B200_GEMM", "auto")
        self.lib.ts_set_pdl.argtypes = [I]
        self.lib.ts_set_pdl.restype = None
        self.lib.ts_set_pdl(0 if os.environ.get("TURINGSERVE_B200_PDL", "1") == "0" else 1)
        self.lib.ts_set_clusters.argtypes = [I]
        self.lib.ts_set_clusters.restype = None
        self.lib.ts_set_clusters(0 if os.environ.get("TURINGSERVE_B200_CLUSTERS", "1") == "0" else 1)
        self.lib.ts_attention_prefill_tc_supported.argtypes = [I, I, I, I, I]
        self.lib.ts_attention_prefill_tc_supported.restype = c_int
        self.lib.ts_attention_prefill_tc_status.argtypes = []
        self.lib.ts_attention_prefill_tc_status.restype = c_int
        # prompt-portion attention on tcgen05 (head size 128, pages of a multiple of 16 tokens) or mma.sync
        self.use_tc_attention = os.environ.get("TURINGSERVE_B200_ATTENTION", "tc") == "tc"
        # its tiles of keys: 64 (two blocks an SM), 128 (one), 0 = by the size of the launch
        self.lib.ts_set_prefill_tile.argtypes = [I]
        self.lib.ts_set_prefill_tile.restype = None
        self.lib.ts_set_prefill_tile(int(os.environ.get("TURINGSERVE_B200_ATTENTION_TILE", "0")))
        self.lib.ts_attention_prefill_supported.argtypes = [I, I, I, I]
        self.lib.ts_attention_prefill_supported.restype = c_int
        for name, args in (("ts_decode_step_max_stages", [I]), ("ts_decode_step_blocks", [I, I]),
                           ("ts_decode_step_work_bytes", [I]), ("ts_decode_step_status", [])):
            getattr(self.lib, name).argtypes = args
            getattr(self.lib, name).restype = c_int
        self.lib.ts_attention_decode_scratch_floats.argtypes = [I, I, I, I]
        self.lib.ts_attention_decode_scratch_floats.restype = ctypes.c_longlong
        self._device_index = torch.cuda.current_device()
        self.num_sms = torch.cuda.get_device_properties(self._device_index).multi_processor_count
        # work buffers by name; one that was outgrown is kept, not freed: a captured graph may still
        # hold its address
        self._buffers: dict[str, torch.Tensor] = {}
        self._outgrown: list[torch.Tensor] = []
        self._decode_slots: dict = {}
        self.use_fast_attention = True
        self.use_fused_step = True          # a whole decode step as one kernel where the model allows it
        self.use_library_gemm = True
        self.max_splits = 10        # (the fused reduce kernels load up to 16 partial sums in one go)
        self.launches = 0           # kernels of this library launched (graph replays add their share)

    # -- plumbing -----------------------------------------------------------------------------------
    def _stream(self) -> int:
        # the raw handle of the current stream: a tenth of the cost of building a torch.cuda.Stream
        # object for it, and every kernel launch asks
        return torch._C._cuda_getCurrentRawStream(self._device_index)

    def _buffer(self, name: str, numel: int, dtype: torch.dtype, device, floor: int = 0, zero: bool = False) -> torch.Tensor:
        """A work buffer of at least ``numel`` elements that lives as long as this object.  When a
        larger one is needed the old one is set aside, never freed: decode graphs captured earlier
        read and write it at its address on every replay."""
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        buf = self._buffers.get(name)
        if buf is None or buf.numel() < numel or buf.device != device:
            if buf is not None:
                self._outgrown.append(buf)
            make = torch.zeros if zero else torch.empty
            buf = self._buffers[name] = make(max(int(numel), floor), dtype=dtype, device=device)
        return buf

    def _check(self, rc: int, what: str) -> None:
        self.launches += 1
        if rc != 0:
            msg = self.lib.ts_last_error().decode(errors="replace")
            raise KernelError(f"{what} failed ({rc}): {msg}")

    # -- kernels ------------------------------------------------------------------------------------
    def embedding(self, out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
        T, h = out.shape
        self._check(self.lib.ts_embedding(_ptr(out), _ptr(table), _ptr(ids), T, h, table.shape[0],
                                          _code(out.dtype), self._stream()), "embedding")

    def gather_rows(self, out: torch.Tensor, x: torch.Tensor, rows: torch.Tensor) -> None:
        S, w = out.shape
        self._check(self.lib.ts_gather_rows(_ptr(out), _ptr(x), _ptr(rows), S, w, _code(x.dtype),
                                            self._stream()), "gather_rows")

    # Up to this many tokens the output and down projections add themselves to the residual stream
    # (their K splits summed by a thread-block cluster) and the norm that follows reads the finished
    # rows: 1.437 -> 1.413 ms a decode step at batch 8, 1.753 -> 1.715 ms at batch 16, 1.966 -> 1.908 ms
    # at batch 32, 2.484 -> 2.402 ms at batch 64.  0: they leave partial sums for the norm kernel.
    fused_link_tokens = int(os.environ.get("TURINGSERVE_B200_FUSED_LINK_TOKENS", "64"))

    def _settle(self, x):
        """What the kernels that finish a split-K sum take: a product not yet launched is launched now,
        its partial sums left in scratch."""
        if isinstance(x, LazyProduct):
            return self.linear(x.out, x.x, x.w, x.bias, may_defer=True, lazy=False)
        return x

    def materialize(self, x):
        """A plain tensor for ``x``, running or finishing what was put off."""
        if isinstance(x, LazyProduct):
            return self.linear(x.out, x.x, x.w, x.bias)
        if not isinstance(x, Deferred):
            return x
        x.out.copy_(x.part[: x.splits].sum(0) if x.bias is None else x.part[: x.splits].sum(0) + x.bias.float())
        return x.out

    def rmsnorm(self, out, x, weight, eps: float, residual=None) -> None:
        """out = weight * norm(x), or of x + residual (which then holds the sum)."""
        if isinstance(x, LazyProduct):
            if residual is not None and self._into_residual(x, residual):
                x, residual = residual, None             # the sum is in place: what is left is a plain norm of it
            else:
                x = self._settle(x)
        self._rmsnorm(out, x, weight, eps, residual)

    def _into_residual(self, p: LazyProduct, residual: torch.Tensor) -> bool:
        """residual += product, in one kernel; False when that kernel does not take the shape."""
        M, N = p.shape
        K = p.w.shape[1]
        if not (residual.dtype == torch.bfloat16 and residual.is_contiguous() and tuple(residual.shape) == (M, N)):
            return False
        splits = min(self.tc_splits(M, N, K), 8)
        if M <= 16 and M > 4 * splits:
            # up to 16 tokens a block of the cluster sums its tokens one after the other: with few splits that
            # are many (0.5B shape, 16 tokens over 3 splits: 1.201 against 1.162 ms a step with the norm kernel)
            return False
        rc = self.lib.ts_linear_tc_resid(_ptr(residual), _ptr(p.x), _ptr(p.w), _ptr(p.bias), M, N, K, splits, self._stream())
        if rc == self.UNSUPPORTED:
            return False
        self._check(rc, "linear_tc_resid")
        return True

    def _rmsnorm(self, out, x, weight, eps: float, residual=None) -> None:
        if isinstance(x, Deferred):
            T, h = x.shape
            if h % 8 == 0 and h <= 16384 and x.dtype == torch.bfloat16:
                self._check(self.lib.ts_reduce_rmsnorm(
                    _ptr(out), _ptr(x.part), x.splits, _ptr(x.bias), _ptr(residual), _ptr(weight), float(eps), T, h,
                    _code(weight.dtype), self._stream()), "reduce_rmsnorm")
                return
            x = self.materialize(x)
        T, h = x.shape
        self._check(self.lib.ts_rmsnorm(_ptr(out), _ptr(x), _ptr(residual), _ptr(weight), float(eps), T, h,
                                        _code(x.dtype), _code(weight.dtype), self._stream()), "rmsnorm")

    def silu_mul(self, out, gu, group: int = 0) -> None:
        """out = silu(gate) * up.  ``group`` 0: gu = [gates | ups]; else gu comes in blocks of
        2 * group columns, group gates then the matching group ups."""
        T, inter = out.shape
        self._check(self.lib.ts_silu_mul_ex(_ptr(out), _ptr(gu), T, inter, group, _code(gu.dtype), self._stream()),
                    "silu_mul")

    GATE_GROUP = 64      # rows of gates, then of ups, in one 128-row tile of the few-token product
    # up to this many tokens the activation goes into the product's epilogue (the kernel takes 128; above
    # 16 tokens all four warps of its epilogue share the activation: 1.739 -> 1.688 ms a step at batch 24,
    # 1.857 -> 1.805 ms at batch 32; at batch 48 and 64 it is within half a percent of the kernel of its own)
    fused_gate_tokens = int(os.environ.get("TURINGSERVE_B200_FUSED_GATE_TOKENS", "32"))

    def gated_linear(self, out, x, w, bias, group: int) -> None:
        """out[T, I] = silu(g) * u with [g, u] = x @ w[2I, K]^T + bias, the rows of ``w`` (and
        ``bias``) laid out as ``silu_mul`` describes.  A few bfloat16 tokens and blocks of 64: one
        kernel, the activation in the product's epilogue; otherwise product, then activation."""
        T, inter = out.shape
        K = w.shape[1]
        use_tc = self.gemm_mode == "tc" or (self.gemm_mode == "auto" and T <= 128)
        if (x.dtype == torch.bfloat16 and use_tc and bias is None and group == self.GATE_GROUP and T <= self.fused_gate_tokens
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            rc = self.lib.ts_linear_tc_gated(_ptr(out), _ptr(x), _ptr(w), T, 2 * inter, K, self._stream())
            if rc != self.UNSUPPORTED:
                self._check(rc, "linear_tc_gated")
                return
        if (x.dtype == torch.bfloat16 and bias is None and group == self.GATE_GROUP and T > self.fused_gate_tokens
                and x.is_contiguous() and self.pair_wins(T, 2 * inter, K, 6.0 * T * inter)
                and self.linear_pair(out, x, w, None, self.PAIR_GATED)):
            return
        gu = torch.empty((T, 2 * inter), dtype=x.dtype, device=x.device)
        self.linear(gu, x, w, bias)
        self.silu_mul(out, gu, group)

    def rope_kv_write(self, qkv, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots,
                      page_size):
        """Rotates q and k in place and writes k, v to the cache; returns the q/k/v tensor.  ``qkv`` may
        be a deferred product: the kernel then finishes its sum on the way."""
        qkv = self._settle(qkv)
        if isinstance(qkv, Deferred):
            d = qkv
            if (self.lib.ts_rope_kv_write_fused_supported(D, rotary_dim, _code(d.dtype))
                    and all(t is None or t.data_ptr() % 16 == 0 for t in (d.out, k_cache, v_cache, cos, sin))):
                self._check(self.lib.ts_rope_kv_write_ex(
                    _ptr(d.out), _ptr(positions), _ptr(cos), _ptr(sin), _ptr(k_cache), _ptr(v_cache), _ptr(slots),
                    d.shape[0], H, KVH, D, rotary_dim, page_size, _code(d.dtype), _ptr(d.part), d.splits,
                    _ptr(d.bias), self._stream()), "rope_kv_write")
                return d.out
            qkv = self.materialize(d)
        T = qkv.shape[0]
        self._check(self.lib.ts_rope_kv_write(
            _ptr(qkv), _ptr(positions), _ptr(cos), _ptr(sin), _ptr(k_cache), _ptr(v_cache), _ptr(slots),
            T, H, KVH, D, rotary_dim, page_size, _code(qkv.dtype), self._stream()), "rope_kv_write")
        return qkv

    # up to this many tokens the q/k/v product finishes itself (sum over its splits, bias, rotation,
    # cache write in its own epilogue) instead of leaving that to the rotary kernel (batch 24: 1.93
    # against 2.09 ms a step; batch 48: 2.12 against 2.27 ms, batch 64: 2.32 against 2.39 ms since the
    # block that finishes a token takes four pairs a thread)
    fused_qkv_tokens = int(os.environ.get("TURINGSERVE_B200_FUSED_QKV_TOKENS", "64"))

    def qkv_rope(self, out, x, w, bias, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots,
                 page_size):
        """out[T, (H + 2 KVH) D] = x @ w^T + bias with q and k rotated, and the new keys and values
        written to the cache: one kernel for a few bfloat16 tokens with heads of 64 or 128 rotated over
        their full width, otherwise the product and then ``rope_kv_write``.  Returns the q/k/v tensor."""
        T, K = x.shape[0], w.shape[1]
        use_tc = self.gemm_mode == "tc" or (self.gemm_mode == "auto" and T <= 128)
        if (x.dtype == torch.bfloat16 and use_tc and T <= self.fused_qkv_tokens and D in (64, 128) and rotary_dim == D
                and cos is not None and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and self.lib.ts_linear_tc_supported(T, (H + 2 * KVH) * D, K)):
            splits = self.tc_splits(T, (H + 2 * KVH) * D, K)
            need = self.lib.ts_linear_tc_qkv_rope_scratch_floats(T, -(-(H + 2 * KVH) * D // 128), splits)
            qkv_part = self._buffer("qkv_part", need, torch.float32, x.device, floor=1 << 18)
            qkv_counters = self._buffer("qkv_counters", 4096, torch.int32, x.device, zero=True)
            if (H + 2 * KVH) * -(-T // 16) <= qkv_counters.numel():
                rc = self.lib.ts_linear_tc_qkv_rope(
                    _ptr(out), _ptr(x), _ptr(w), _ptr(bias), _ptr(qkv_part), _ptr(qkv_counters),
                    _ptr(positions), _ptr(cos), _ptr(sin), _ptr(slots), _ptr(k_cache), _ptr(v_cache), T, H, KVH, D,
                    page_size, K, splits, self._stream())
                if rc != self.UNSUPPORTED:
                    self._check(rc, "linear_tc_qkv_rope")
                    return out
        if (self.pair_qkv and T > self.fused_qkv_tokens and x.dtype == torch.bfloat16 and D in (64, 128) and rotary_dim == D
                and cos is not None and cos.dtype == torch.float32 and x.is_contiguous()
                and self.pair_wins(T, (H + 2 * KVH) * D, K, 4.0 * T * (H + 2 * KVH) * D)):
            x = self.materialize(x)
            rc = self.lib.ts_linear_pair_qkv(
                _ptr(out), _ptr(x), _ptr(w), _ptr(bias), _ptr(positions), _ptr(cos), _ptr(sin), _ptr(slots),
                _ptr(k_cache), _ptr(v_cache), T, H, KVH, D, page_size, K, self._stream())
            if rc != self.UNSUPPORTED:
                self._check(rc, "linear_pair_qkv")
                return out
        qkv = self.linear(out, x, w, bias, may_defer=True)
        return self.rope_kv_write(qkv, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots, page_size)

    def scratch(self, floats: int, device) -> torch.Tensor:
        """A float32 work buffer of at least ``floats`` elements, kept between calls."""
        return self._buffer("scratch", floats, torch.float32, device, floor=1 << 20)

    def decode_splits(self, num_requests: int, KVH: int, max_seq_len: int) -> int:
        """How many pieces each request's keys are cut into so that the launch fills the GPU
        (the cp.async decode kernel: two blocks per SM, pieces of at least 256 keys)."""
        want = -(-2 * self.num_sms // max(1, num_requests * KVH))
        return max(1, min(want, -(-max_seq_len // 256), 128))

    def decode_splits_tma(self, num_requests: int, KVH: int, D: int, max_seq_len: int) -> int:
        """The most pieces a request's keys may be cut into by the TMA decode kernel, which deals
        tiles of 64 keys out evenly over as many of them as get a tile: as many as one wave of
        blocks holds (the kernel itself uses fewer when the contexts are short)."""
        key = (D, self.decode_stages)
        if key not in self._decode_slots:
            self._decode_slots[key] = max(1, self.lib.ts_attention_decode_tma_blocks_per_sm(D, self.decode_stages))
        slots = self.num_sms * self._decode_slots[key]
        pairs = max(1, num_requests * KVH)
        tiles = max(1, -(-max_seq_len // 64))
        return max(1, min(slots // pairs, tiles, 128))

    def _decode_scratch(self, nd: int, H: int, KVH: int, D: int, nsplit: int, device):
        if nsplit <= 1:
            return None, None
        scratch = self.scratch(self.lib.ts_attention_decode_scratch_floats(nd, H, D, nsplit), device)
        # (one ticket counter per (request, kv head); the streaming kernel's two-level merge of more than 16
        # splits takes 16 more for each)
        return scratch, self._buffer("counters", nd * KVH * 17, torch.int32, device, floor=1 << 16, zero=True)

    def attention(self, out, qkv, k_cache, v_cache, block_tables, step, H, KVH, D, page_size, scale,
                  window) -> None:
        """Rows of requests with one token (the first ``step.num_decode`` requests) go to a
        split-key decode kernel when one takes the shape; the rest to the chunk kernels."""
        w = 0 if window is None else int(window)
        code = _code(qkv.dtype)
        B, nd = step.num_requests, 0
        width = block_tables.shape[1]
        streaming = self.decode_kernel == "tma"
        if self.decode_kernel == "auto":
            streaming = getattr(step, "streaming_decode", None)
            if streaming is None:
                streaming = step.num_decode * step.max_seq_len >= 98304
            # The other kernel is the faster one only while its blocks of 8 warps fit one per SM, eight to
            # a (request, kv head): from ten requests with two kv heads on, the streaming kernel wins at
            # every context (batch 12 x 2,048 keys: 12.3 against 18.7 us; batch 16 x 256 keys: 9.5 against 12.8)
            streaming = streaming or step.num_decode * KVH * 8 > self.num_sms
        if (self.use_fast_attention and streaming and step.num_decode > 0
                and self.lib.ts_attention_decode_tma_supported(H, KVH, D, page_size, code)):
            nd = step.num_decode
            nsplit = self.decode_splits_tma(nd, KVH, D, step.max_seq_len)
            scratch, counters = self._decode_scratch(nd, H, KVH, D, nsplit, qkv.device)
            rc = self.lib.ts_attention_decode_tma(
                _ptr(out), _ptr(scratch), _ptr(counters), _ptr(qkv), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                _ptr(step.q_start), _ptr(step.seq_lens), nd, width, H, KVH, D, page_size, k_cache.shape[0],
                float(scale), w, nsplit, self.decode_stages, self._stream())
            if rc == self.UNSUPPORTED:          # e.g. key and value caches that no one tensor map spans
                nd = 0
            else:
                self._check(rc, "attention_decode_tma")
        if nd == 0 and self.use_fast_attention and step.num_decode > 0 and self.lib.ts_attention_decode_supported(H, KVH, D, code):
            nd = step.num_decode
            nsplit = self.decode_splits(nd, KVH, step.max_seq_len)
            scratch, counters = self._decode_scratch(nd, H, KVH, D, nsplit, qkv.device)
            self._check(self.lib.ts_attention_decode(
                _ptr(out), _ptr(scratch), _ptr(counters), _ptr(qkv), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                _ptr(step.q_start), _ptr(step.seq_lens), nd, width, H, KVH, D, page_size, float(scale), w,
                nsplit, self._stream()), "attention_decode")
        if nd == B:
            return
        if (self.use_fast_attention and self.use_tc_attention
                and self.lib.ts_attention_prefill_tc_supported(H, KVH, D, page_size, code)):
            self._check(self.lib.ts_attention_prefill_tc(
                _ptr(out), _ptr(qkv), _ptr(k_cache), _ptr(v_cache), block_tables.data_ptr() + 4 * nd * width,
                step.q_start.data_ptr() + 4 * nd, step.seq_lens.data_ptr() + 4 * nd, B - nd, width,
                step.max_q_len, H, KVH, D, page_size, k_cache.shape[0], float(scale), w, self._stream()),
                "attention_prefill_tc")
            return
        if self.use_fast_attention and self.lib.ts_attention_prefill_supported(H, KVH, D, code):
            self._check(self.lib.ts_attention_prefill(
                _ptr(out), _ptr(qkv), _ptr(k_cache), _ptr(v_cache), block_tables.data_ptr() + 4 * nd * width,
                step.q_start.data_ptr() + 4 * nd, step.seq_lens.data_ptr() + 4 * nd, B - nd, width,
                step.max_q_len, H, KVH, D, page_size, float(scale), w, self._stream()), "attention_prefill")
            return
        self._check(self.lib.ts_attention_generic(
            _ptr(out), _ptr(qkv), _ptr(k_cache), _ptr(v_cache), block_tables.data_ptr() + 4 * nd * width,
            step.q_start.data_ptr() + 4 * nd, step.seq_lens.data_ptr() + 4 * nd, B - nd, width,
            step.max_q_len, H, KVH, D, page_size, float(scale), w, code, self._stream()), "attention")

    def linear(self, out, x, w, bias=None, rows=None, may_defer: bool = False, lazy: bool = True):
        """out[M, N] = x[rows or all, :] @ w[N, K]^T + bias.  Returns ``out``; or, when ``may_defer``
        and the few-token tensor-core kernel takes the product, a ``LazyProduct`` (not launched yet:
        the norm that gets it with a residual launches it fused with the residual add) or a ``Deferred``
        whose sum the consuming norm finishes (``out`` is then left untouched)."""
        M, N = out.shape
        K = w.shape[1]
        x = self.materialize(x)
        use_tc = self.gemm_mode == "tc" or (self.gemm_mode == "auto" and M <= 128)
        if (may_defer and lazy and rows is None and use_tc and x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                and 0 < M <= self.fused_link_tokens and self.lib.ts_linear_tc_supported(M, N, K)
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            return LazyProduct(out, x, w, bias)
        if x.dtype == torch.bfloat16 and (use_tc or self.use_library_gemm) and rows is not None:
            xg = torch.empty((M, K), dtype=x.dtype, device=x.device)
            self.gather_rows(xg, x, rows)
            x, rows = xg, None
        if (x.dtype == torch.bfloat16 and use_tc and self.lib.ts_linear_tc_supported(M, N, K)
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            splits = self.tc_splits(M, N, K)
            if may_defer and M <= 128 and N % 8 == 0 and out.dtype == torch.bfloat16:
                part = self.partial_scratch(splits * M * N, x.device)
                used = ctypes.c_int(0)
                self._check(self.lib.ts_linear_tc_ex(_ptr(out), _ptr(x), _ptr(w), None, _ptr(part), M, N, K, 0, splits,
                                                     1, ctypes.addressof(used), self._stream()), "linear_tc")
                return Deferred(part.view(-1)[: used.value * M * N].view(used.value, M, N), used.value, (M, N),
                                out.dtype, bias, out)
            scratch = self.scratch(splits * M * N, x.device) if splits > 1 else None
            self._check(self.lib.ts_linear_tc(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), _ptr(scratch), M, N, K,
                                              1 if out.dtype == torch.float32 else 0, splits, self._stream()),
                        "linear_tc")
            if splits > 1:
                self.launches += 1
            return out
        if x.dtype == torch.bfloat16 and self.use_library_gemm:
            if out.dtype == torch.float32:
                torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
                if bias is not None:
                    out.add_(bias.float())
            elif bias is not None:
                torch.addmm(bias, x, w.t(), out=out)
            else:
                torch.mm(x, w.t(), out=out)
            return out
        self._check(self.lib.ts_linear_simt(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), _ptr(rows), M, N, K,
                                            _code(x.dtype), _code(out.dtype), self._stream()), "linear")
        return out

    # -- a residual stream in 32-bit ---------------------------------------------------------------------
    def rmsnorm_stream(self, out, stream, add1, add2, weight, eps: float, first: bool = False, alpha: float = 1.0,
                       row=None, norm_bias=None) -> None:
        """stream (float32 [T, h]) += alpha * (add1 + add2) + row (add1, add2 and ``row``, a float32 [h] vector
        common to all tokens, may be None; ``first``: the stream is started from them instead);
        out = stream / sqrt(mean(stream^2) + eps) * weight, or with ``norm_bias`` the layer norm
        (stream - mean) / sqrt(variance + eps) * weight + norm_bias; 32-bit, rounded once.  ``out`` None: only the sum."""
        T, h = stream.shape
        part, splits, bias = None, 0, None
        if isinstance(add1, (LazyProduct, Deferred)) and self.lib.ts_rmsnorm_wide_takes_parts(h):
            # a few-token product that was put off: its partial sums are summed here, no kernel of their own
            add1 = self._settle(add1)
            if isinstance(add1, Deferred) and add1.part.data_ptr() % 16 == 0 and stream.data_ptr() % 16 == 0:
                part, splits, bias, dt = add1.part, add1.splits, add1.bias, add1.dtype
                add1 = None
        add1, add2 = self.materialize(add1), self.materialize(add2)
        if part is None:
            dt = add1.dtype if add1 is not None else (add2.dtype if add2 is not None else out.dtype)
        self._check(self.lib.ts_rmsnorm_wide(_ptr(out), _ptr(stream), _ptr(add1), _ptr(add2), _ptr(weight), float(eps),
                                             T, h, 1 if first else 0, _code(dt), _code(weight.dtype), _ptr(part), splits,
                                             _ptr(bias), float(alpha), _ptr(row), _ptr(norm_bias), self._stream()),
                    "rmsnorm_stream")

    def gated_rmsnorm(self, out, x, gate, weight, eps: float) -> None:
        """out = x / sqrt(mean(x^2) + eps) * weight * sigmoid(gate), x float32 [T, n]; ``gate`` [T, n] in
        out's type, possibly a column slice of a wider tensor."""
        T, n = x.shape
        if gate.stride(1) != 1:
            raise ValueError("gated_rmsnorm: the gate's rows must be contiguous")
        self._check(self.lib.ts_gated_rmsnorm(_ptr(out), _ptr(x), _ptr(gate), gate.stride(0), _ptr(weight), float(eps), T,
                                              n, _code(out.dtype), _code(weight.dtype), self._stream()), "gated_rmsnorm")

    diff_decode_splits = int(os.environ.get("TURINGSERVE_B200_DIFF_DECODE_SPLITS", "16"))

    ACTIVATIONS = {"none": 0, "gelu_tanh": 1, "relu2": 2, "silu": 3, "gelu": 4}

    def activation(self, out, x, kind: str) -> None:
        """out = act(x) elementwise (32-bit arithmetic, one rounding); out may be x.  ``x`` may be a product that
        was put off: its partial sums are summed on the way."""
        x = self._settle(x)
        if isinstance(x, Deferred):
            rows, cols = x.shape
            self._check(self.lib.ts_activation_parts(_ptr(out), _ptr(x.part), x.splits, _ptr(x.bias), rows, cols,
                                                     self.ACTIVATIONS[kind], _code(out.dtype), self._stream()),
                        "activation_parts")
            return
        self._check(self.lib.ts_activation(_ptr(out), _ptr(x), x.numel(), self.ACTIVATIONS[kind], _code(x.dtype),
                                           self._stream()), "activation")

    # -- linear attention with a decaying matrix state ----------------------------------------------------
    def lightning(self, out, proj, state, decay, step, H: int, D: int, V: int) -> None:
        """out (float32 [T, H V]): per head o_t = S_t^T q_t with S_t = decay_h S_(t-1) + k_t v_t^T, where
        q, k, v = silu of the columns [0, HD), [HD, 2HD), [2HD, 2HD + HV) of ``proj``; ``state``
        (float32 [slots, H, D, V]) is read and left updated at each request's slot."""
        self._check(self.lib.ts_lightning_ex(_ptr(out), _ptr(proj), proj.stride(0), _ptr(state), _ptr(decay),
                                             _ptr(step.q_start), _ptr(step.state_slots), step.num_requests, H, D, V,
                                             int(getattr(step, "max_q_len", 0) or 0), _code(proj.dtype), self._stream()),
                    "lightning")

    # -- attention with two score maps a head --------------------------------------------------------------
    def kv_write_pair(self, proj, k_off: int, v_off: int, k_cache, v_cache, slots, KVH: int, DK: int, DV: int,
                      page_size: int) -> None:
        """The step's new key rows (columns k_off.. of ``proj``, KVH x DK) and value rows (v_off.., KVH x DV)
        into their cache slots; a slot of -1 writes nothing."""
        self._check(self.lib.ts_kv_write_pair(_ptr(proj), proj.stride(0), k_off, v_off, _ptr(k_cache), _ptr(v_cache),
                                              _ptr(slots), proj.shape[0], KVH, DK, DV, page_size, _code(proj.dtype),
                                              self._stream()), "kv_write_pair")

    def attention_diff(self, out, proj, k_cache, v_cache, block_tables, step, H: int, KVH: int, D: int, V: int,
                       page_size: int, scale: float, lam: float, eps: float, out_scale: float) -> None:
        """out [T, H V] = out_scale * rmsnorm_head(a1 - lam a2): two causal softmax maps a head (queries in
        the first H 2D columns of ``proj`` as [map 1 | map 2] per head, cached key rows 2D wide) over the
        same cached values.  bfloat16 with maps of 32 or 64 and values of 64 or 128: the tensor-core kernel;
        anything else: the any-size kernel."""
        if (self.use_fast_attention and proj.dtype == torch.bfloat16
                and self.lib.ts_attention_diff_mma_supported(H, KVH, D, V, _code(proj.dtype))):
            # requests that bring one token have their keys cut over so many blocks that every SM has two, sixteen
            # at most (every piece is one more partial result for the last block to fold)
            B = step.num_requests
            splits = max(1, min(self.diff_decode_splits, 2 * self.num_sms // max(1, B * KVH)))
            # which of the kernel's two instances the step needs (the host knows every request's token count)
            q_lens = getattr(step, "q_lens", None)
            G = H // KVH
            kinds = 3 if q_lens is None else ((1 if any(n * G <= 16 for n in q_lens) else 0)
                                              | (2 if any(n * G > 16 for n in q_lens) else 0))
            scratch = counters = None
            if splits > 1:
                scratch = self._buffer("diff_scratch", self.lib.ts_attention_diff_mma_scratch_floats(B, KVH, V, splits),
                                       torch.float32, proj.device, floor=1 << 20)
                counters = self._buffer("diff_counters", B * KVH, torch.int32, proj.device, floor=1 << 12, zero=True)
            rc = self.lib.ts_attention_diff_mma(
                _ptr(out), _ptr(proj), proj.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                _ptr(step.q_start), _ptr(step.seq_lens), B, block_tables.shape[1], step.max_q_len, H,
                KVH, D, V, page_size, float(scale), float(lam), float(eps), float(out_scale), _ptr(scratch),
                _ptr(counters), splits, kinds, self._stream())
            if rc != self.UNSUPPORTED:
                self._check(rc, "attention_diff_mma")
                return
        self._check(self.lib.ts_attention_diff(
            _ptr(out), _ptr(proj), proj.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(step.q_start),
            _ptr(step.seq_lens), step.num_requests, block_tables.shape[1], step.max_q_len, H, KVH, D, V, page_size,
            float(scale), float(lam), float(eps), float(out_scale), _code(proj.dtype), self._stream()), "attention_diff")

    # -- the gated delta rule --------------------------------------------------------------------------------------
    def delta_prepare(self, ready, proj, conv_w, a_log, dt_bias, state, step, H: int, G: int, D: int, V: int, taps: int,
                      unit_eps: float) -> None:
        """ready (float32 [T, 2GD + HV + 2H + G]) = [q | k | v | g | beta | k.q] of every token: the columns q, k, v of
        ``proj`` through their causal filters (``conv_w`` float32 [2GD + HV, taps]; inputs before the step's first
        token come from the request's state slot) and SiLU, q and k to unit length per head and q / sqrt(D),
        g = exp(-exp(a_log) softplus(a + dt_bias)), beta = sigmoid(b); b and a are the last 2H columns of ``proj``."""
        T = proj.shape[0]
        self._check(self.lib.ts_delta_prepare(_ptr(ready), _ptr(proj), proj.stride(0), _ptr(conv_w), _ptr(a_log),
                                              _ptr(dt_bias), _ptr(state), state.stride(0), _ptr(step.token_request),
                                              _ptr(step.q_start), _ptr(step.state_slots), T, H, G, D, V, taps,
                                              float(unit_eps), _code(proj.dtype), self._stream()), "delta_prepare")

    def delta_scan(self, out, ready, proj, state, step, H: int, G: int, D: int, V: int, taps: int) -> None:
        """out (float32 [T, HV]): the recurrence over the rows ``delta_prepare`` made; ``state`` (float32
        [slots, HDV + (taps - 1)(2GD + HV)]) is read and left updated at each request's slot, the filter's last
        inputs (from ``proj``) included."""
        self._check(self.lib.ts_delta_scan(_ptr(out), _ptr(ready), _ptr(proj), proj.stride(0), _ptr(state), state.stride(0),
                                           _ptr(step.q_start), _ptr(step.state_slots), step.num_requests, H, G, D, V, taps,
                                           int(getattr(step, "max_q_len", 0) or 0), _code(proj.dtype), self._stream()), "delta_scan")

    def head_gated_rmsnorm(self, out, x, gate, weight, eps: float, H: int, V: int) -> None:
        """out [T, HV] = x / rms over each head's V * weight[V] * silu(gate); x float32; ``gate`` possibly a column
        slice of a wider tensor."""
        if gate.stride(1) != 1:
            raise ValueError("head_gated_rmsnorm: the gate's rows must be contiguous")
        self._check(self.lib.ts_head_gated_rmsnorm(_ptr(out), _ptr(x), _ptr(gate), gate.stride(0), _ptr(weight), float(eps),
                                                   x.shape[0], H, V, _code(out.dtype), self._stream()), "head_gated_rmsnorm")

    # -- norms, rotations and per-head products around an attention ----------------------------------------------------
    def rms_rows(self, out, x, col0: int, weight, eps: float) -> None:
        """out [T, n] = rms norm of the columns col0 .. col0 + n of ``x`` times ``weight`` (float32)."""
        T, n = out.shape
        self._check(self.lib.ts_rms_rows(_ptr(out), _ptr(x), x.stride(0), col0, n, _ptr(weight), float(eps), T,
                                         _code(x.dtype), self._stream()), "rms_rows")

    def qk_rownorm_write(self, proj, q_w, k_w, eps: float, positions, coef: float, every: int, k_cache, v_cache, slots,
                         H: int, G: int, D: int, page_size: int) -> None:
        """``proj`` [T, (H + G) D] = [q | k]: q normed over its whole row, times ``q_w`` and the temperature
        1 + coef ln(floor((p + 1) / every) + 1), in place; k normed over its whole row times ``k_w`` into ``k_cache``
        and k as projected into ``v_cache`` at ``slots`` (None: nothing is cached)."""
        self._check(self.lib.ts_qk_rownorm_write(_ptr(proj), proj.stride(0), _ptr(q_w), _ptr(k_w), float(eps), _ptr(positions),
                                                 float(coef), int(every), _ptr(k_cache), _ptr(v_cache), _ptr(slots),
                                                 proj.shape[0], H, G, D, page_size, _code(proj.dtype), self._stream()),
                    "qk_rownorm_write")

    def latent_kv_write(self, proj, col0: int, weight, eps: float, positions, freq, magnitude: float, rot_dims: int, k_cache,
                        slots, rank: int, R: int, page_size: int) -> None:
        """The cached row of every token, [rms(latent) * weight | rotated key part], from the columns col0 .. of
        ``proj`` into ``k_cache`` [pages, 1, page, rank + R] at ``slots``."""
        self._check(self.lib.ts_latent_kv_write(_ptr(proj), proj.stride(0), col0, _ptr(weight), float(eps), _ptr(positions),
                                                _ptr(freq), float(magnitude), rot_dims, _ptr(k_cache), _ptr(slots),
                                                proj.shape[0], rank, R, page_size, _code(proj.dtype), self._stream()),
                    "latent_kv_write")

    def rotate_pairs(self, dst, src, positions, freq, magnitude: float, rot_dims: int) -> None:
        """dst[t, h, :] = src[t, h, :] with its first ``rot_dims`` dimensions rotated in neighbouring pairs by
        position * freq[i] (cosine and sine times ``magnitude``); [T, H, R] views with unit last stride."""
        T, H, R = src.shape
        if dst.stride(2) != 1 or src.stride(2) != 1:
            raise ValueError("rotate_pairs: rows must be contiguous")
        self._check(self.lib.ts_rotate_pairs(_ptr(dst), dst.stride(0), dst.stride(1), _ptr(src), src.stride(0), src.stride(1),
                                             _ptr(positions), _ptr(freq), float(magnitude), rot_dims, T, H, R,
                                             _code(src.dtype), self._stream()), "rotate_pairs")

    def rope_headnorm_write(self, proj, k_off: int, v_off: int, positions, freq, rot_dims: int, norm_eps, k_cache, v_cache,
                            slots, H: int, G: int, D: int, V: int, page_size: int):
        """``proj`` [T, ...]: q heads in the columns [0, H D), k heads from ``k_off``, value rows from ``v_off``.  Every q and
        k head has dimension i < rot_dims / 2 turned with dimension i + rot_dims / 2 by position * freq[i] (32-bit) and,
        with ``norm_eps`` not None, is then divided by its root mean square (eps inside the root, no weight); q in place,
        k into ``k_cache`` and the value rows into ``v_cache`` at ``slots`` (None: nothing is cached).  ``proj`` may be a
        product put off: the kernel then finishes its sum on the way (of the returned tensor only the q columns are
        written).  Returns the projection tensor."""
        proj = self._settle(proj)
        part, splits = None, 0
        if isinstance(proj, Deferred):
            d = proj
            if (d.bias is None and int(rot_dims) % 16 == 0
                    and self.lib.ts_rope_headnorm_write_supports_parts(d.out.stride(0), k_off, D, _code(d.dtype))
                    and all(t is None or t.data_ptr() % 16 == 0 for t in (d.out, d.part, k_cache))):
                part, splits, proj = d.part, d.splits, d.out
            else:
                proj = self.materialize(d)
        self._check(self.lib.ts_rope_headnorm_write(
            _ptr(proj), proj.stride(0), k_off, v_off, _ptr(positions), _ptr(freq), int(rot_dims), 0 if norm_eps is None else 1,
            float(norm_eps or 0.0), _ptr(k_cache), _ptr(v_cache), _ptr(slots), proj.shape[0], H, G, D, V, page_size,
            _code(proj.dtype), _ptr(part), splits, self._stream()), "rope_headnorm_write")
        return proj

    # bfloat16 per-head products with at least this many rows go to the library's batched product
    batched_library_rows = int(os.environ.get("TURINGSERVE_B200_BATCHED_LIBRARY_ROWS", "17"))

    def batched_linear(self, out, x, w) -> None:
        """out[t, h, :] = w[h] x[t, h, :]: ``x`` [T, H, K] and ``out`` [T, H, N] views with unit last stride,
        ``w`` [H, N, K] contiguous.  This library's kernels (up to 16 rows: a warp an output column, streaming
        its weight row; float32 above: FFMA tiles, fixed k order); bfloat16 with more rows: the vendor's batched product."""
        T, H, K = x.shape
        N = w.shape[1]
        if out.stride(2) != 1 or x.stride(2) != 1 or not w.is_contiguous():
            raise ValueError("batched_linear: rows must be contiguous")
        if x.dtype == torch.bfloat16 and self.use_library_gemm and T >= self.batched_library_rows:
            torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))
            return
        self._check(self.lib.ts_batched_linear(_ptr(out), out.stride(0), out.stride(1), _ptr(x), x.stride(0), x.stride(1),
                                               _ptr(w), T, H, N, K, _code(x.dtype), self._stream()), "batched_linear")

    biased_decode_splits = int(os.environ.get("TURINGSERVE_B200_BIASED_DECODE_SPLITS", "0"))

    def attention_biased(self, out, q, k_cache, v_cache, block_tables, step, KVH: int, page_size: int, scale: float,
                         softcap: float, slopes, window, chunk=None, sinks=None) -> None:
        """out [T, H, Dv] = softmax over the visible keys of cap tanh(q.k scale / cap) - slope_h (i - j), times the
        values; q [T, H, Dk] (views with unit last stride).  ``v_cache`` None: the values are the first Dv columns
        of the key rows.  ``softcap`` 0: none; ``slopes`` (float32 [H]) None: none; ``window`` None: none; ``chunk`` c:
        position i sees only j >= floor(i / c) c; ``sinks`` (float32 [H]): exp(sink_h) joins the softmax's denominator.  The keys
        of requests that bring one token are cut over several blocks when the step's longest context is long."""
        T, H, Dk = q.shape
        Dv = out.shape[2]
        if out.stride(2) != 1 or q.stride(2) != 1:
            raise ValueError("attention_biased: rows must be contiguous")
        B = step.num_requests
        w = 0 if window is None else int(window)
        reach = min(step.max_seq_len, w) if w else step.max_seq_len
        c = 0 if chunk is None else int(chunk)
        if c:
            reach = min(reach, c)
        splits = self.biased_decode_splits
        v_in_k = 1 if v_cache is None else 0
        if (self.use_fast_attention and q.dtype == torch.bfloat16
                and self.lib.ts_attention_biased_mma_supported(H, KVH, Dk, Dv, v_in_k, _code(q.dtype))):
            # the tensor-core kernel: key rows of 64, 128 (values of the same width) or latent rows with the values inside
            chunks = Dv // self.lib.ts_attention_biased_mma_chunk(Dk, Dv, v_in_k)
            nd, G = step.num_decode, H // KVH
            width = block_tables.shape[1]
            # Requests that bring one token: their keys cut over blocks.  Where a kv head serves at most 32 heads they go
            # to an instance whose warps share every tile's keys (a launch of their own, four or two partial results a
            # block); else they ride in the other requests' launch, with the warps that have no rows idle.
            spread = nd > 0 and G <= 32
            ms = 1
            if nd > 0 and G <= 64:
                ms = max(1, min(16, (8 if spread else 16) if splits <= 0 else splits,
                                2 * self.num_sms // max(1, nd * KVH * chunks), reach // (256 if spread else 128)))

            def launch(first: int, count: int, max_q: int, n_splits: int, spread_flag: int) -> int:
                scratch = counters = None
                if n_splits > 1 or spread_flag:
                    scratch = self._buffer("biased_mma_scratch",
                                           self.lib.ts_attention_biased_mma_scratch_floats(count, KVH, Dk, Dv, v_in_k, n_splits),
                                           torch.float32, q.device, floor=1 << 20)
                    counters = self._buffer("biased_mma_counters", count * KVH * chunks, torch.int32, q.device, floor=1 << 14,
                                            zero=True)
                return self.lib.ts_attention_biased_mma(
                    _ptr(out), out.stride(0), out.stride(1), _ptr(q), q.stride(0), q.stride(1), _ptr(k_cache), _ptr(v_cache),
                    block_tables.data_ptr() + 4 * first * width, step.q_start.data_ptr() + 4 * first,
                    step.seq_lens.data_ptr() + 4 * first, count, width, max_q, H, KVH, Dk, Dv, page_size, float(scale),
                    float(softcap), _ptr(slopes), w, n_splits, _ptr(scratch), _ptr(counters), spread_flag, c, _ptr(sinks),
                    self._stream())

            if spread:
                rc = launch(0, nd, 1, ms, 1)
                if rc == 0 and nd < B:
                    self.launches += 1
                    rc = launch(nd, B - nd, step.max_q_len, 1, 0)
            else:
                rc = launch(0, B, step.max_q_len, ms, 0)
            if rc != self.UNSUPPORTED:
                self._check(rc, "attention_biased_mma")
                return
        if splits <= 0:
            # single-token requests: so many pieces that the chip has two blocks an SM, each with four tiles or more
            splits = 1
            if step.num_decode > 0:
                splits = max(1, min(32, 2 * self.num_sms // max(1, step.num_decode * KVH), reach // 128))
        scratch = counters = None
        if splits > 1:
            scratch = self._buffer("biased_scratch", self.lib.ts_attention_biased_scratch_floats(B, KVH, H, step.max_q_len, Dv, splits),
                                   torch.float32, q.device, floor=1 << 20)
            tiles = -(-(step.max_q_len * (H // KVH)) // 16)
            counters = self._buffer("biased_counters", B * KVH * tiles, torch.int32, q.device, floor=1 << 14, zero=True)
        self._check(self.lib.ts_attention_biased(
            _ptr(out), out.stride(0), out.stride(1), _ptr(q), q.stride(0), q.stride(1), _ptr(k_cache), _ptr(v_cache),
            _ptr(block_tables), _ptr(step.q_start), _ptr(step.seq_lens), B, block_tables.shape[1], step.max_q_len, H, KVH,
            Dk, Dv, page_size, float(scale), float(softcap), _ptr(slopes), w, splits, _ptr(scratch), _ptr(counters),
            _code(q.dtype), c, _ptr(sinks), self._stream()), "attention_biased")

    # -- a residual stream in several copies -------------------------------------------------------------------
    def hyper_norm(self, out, streams, y, mix, out_w, in_w, weight, eps: float, first: bool = False,
                   alpha: float = 1.0) -> None:
        """The norm of a residual stream kept as S copies (``streams`` float32 [T, S, h], updated in place).  First the
        pending write-back of a sublayer's output ``y`` ([T, h]; a product put off is summed on the way; None: nothing
        pending): x_t <- sum_s mix[s, t] x_s + out_w[t] y (``first``: every copy starts as alpha * y instead); then
        u = sum_s in_w[s] x_s (``in_w`` None: the plain sum) and out = u / sqrt(mean(u^2) + eps) * weight (``out`` None:
        only the write-back).  ``mix`` [S, S], ``out_w`` [S], ``in_w`` [S], ``weight`` [h]: float32 on the device;
        ``mix`` / ``out_w`` None: identity / ones."""
        T, S, h = streams.shape
        part, splits, bias = None, 0, None
        if isinstance(y, (LazyProduct, Deferred)):
            y = self._settle(y)
            if isinstance(y, Deferred):
                part, splits, bias, dt = y.part, y.splits, y.bias, y.dtype
                y = None
        y = self.materialize(y)
        if part is None:
            dt = y.dtype if y is not None else out.dtype
        self._check(self.lib.ts_hyper_norm(_ptr(out), _ptr(streams), _ptr(y), _ptr(part), splits, _ptr(bias), _ptr(mix),
                                           _ptr(out_w), _ptr(in_w), _ptr(weight), float(eps), T, S, h, 1 if first else 0,
                                           float(alpha), _code(dt), self._stream()), "hyper_norm")

    # -- state-space mixer ---------------------------------------------------------------------------------------
    def ssm_prepare(self, ready, proj, xbc_off: int, dt_off: int, conv_w, conv_b, a_log, dt_bias, state, tail_off: int,
                    step, H: int, channels: int, taps: int) -> None:
        """ready (float32 [T, channels + 2 H]) = [filtered channels | dt | a]: the ``channels`` columns of ``proj``
        from ``xbc_off`` through their causal filters (``conv_w`` float32 [channels, taps], ``conv_b`` [channels]; the
        inputs before the step's first token come from the request's state slot, from ``tail_off`` on) and SiLU;
        dt = softplus(proj[dt_off + h] + dt_bias[h]), a = exp(-exp(a_log[h]) dt)."""
        T = proj.shape[0]
        self._check(self.lib.ts_ssm_prepare(_ptr(ready), _ptr(proj), proj.stride(0), xbc_off, dt_off, _ptr(conv_w),
                                            _ptr(conv_b), _ptr(a_log), _ptr(dt_bias), _ptr(state), state.stride(0),
                                            int(tail_off), _ptr(step.token_request), _ptr(step.q_start),
                                            _ptr(step.state_slots), T, H, channels, taps, _code(proj.dtype),
                                            self._stream()), "ssm_prepare")

    def ssm_scan(self, out, ready, proj, xbc_off: int, state, skip, step, H: int, G: int, N: int, P: int, taps: int) -> None:
        """out (float32 [T, H P]): per head S <- a S + dt B x^T, y = S^T C + skip_h x over the rows ``ssm_prepare`` made;
        ``state`` (float32 [slots, H N P + (taps - 1) channels]) is read and left updated at each request's slot, the
        filter's last inputs (from ``proj``) included."""
        self._check(self.lib.ts_ssm_scan(_ptr(out), _ptr(ready), _ptr(proj), proj.stride(0), xbc_off, _ptr(state),
                                         state.stride(0), _ptr(skip), _ptr(step.q_start), _ptr(step.state_slots),
                                         step.num_requests, H, G, N, P, taps, int(getattr(step, "max_q_len", 0) or 0),
                                         _code(proj.dtype), self._stream()), "ssm_scan")

    GATES = {"sigmoid": 0, "silu": 1}

    def gated_group_rmsnorm(self, out, x, gate, weight, eps: float, groups: int = 1, gate_kind: str = "sigmoid",
                            gate_first: bool = False, scale: float = 1.0) -> None:
        """out [T, n] = RMS norm of ``x`` (float32 [T, n]) in ``groups`` equal parts, each by its own root mean square,
        times ``weight`` (float32 [n]) and ``scale``; the gate (sigmoid or silu of ``gate``) multiplies what is normed
        (``gate_first``) or the result.  ``out`` and ``gate`` may be column slices of wider tensors."""
        T, n = x.shape
        if gate.stride(1) != 1 or out.stride(1) != 1:
            raise ValueError("gated_group_rmsnorm: rows must be contiguous")
        self._check(self.lib.ts_gated_group_rmsnorm(_ptr(out), out.stride(0), _ptr(x), _ptr(gate), gate.stride(0),
                                                    _ptr(weight), float(eps), T, n, int(groups), self.GATES[gate_kind],
                                                    1 if gate_first else 0, float(scale), _code(out.dtype),
                                                    self._stream()), "gated_group_rmsnorm")

    def gate_mul(self, out, a, gate, gate_kind: str = "sigmoid", scale: float = 1.0) -> None:
        """out = a * gate_fn(gate) * scale elementwise over [T, n] views with unit last stride (out may be a)."""
        T, n = a.shape
        if out.stride(1) != 1 or a.stride(1) != 1 or gate.stride(1) != 1:
            raise ValueError("gate_mul: rows must be contiguous")
        self._check(self.lib.ts_gate_mul(_ptr(out), out.stride(0), _ptr(a), a.stride(0), _ptr(gate), gate.stride(0), T, n,
                                         self.GATES[gate_kind], float(scale), _code(a.dtype), self._stream()), "gate_mul")

    def act_mul(self, out, gu, act: str, group: int = 0) -> None:
        """out = act(gate) * up, the columns of ``gu`` laid out as ``silu_mul`` describes; ``act`` a one-input activation."""
        T, inter = out.shape
        self._check(self.lib.ts_act_mul(_ptr(out), _ptr(gu), T, inter, group, self.ACTIVATIONS[act], _code(gu.dtype),
                                        self._stream()), "act_mul")

    def rope_pairs_write(self, proj, k_off: int, v_off: int, positions, freq, magnitude: float, rot_dims: int, k_cache,
                         v_cache, slots, H: int, G: int, D: int, V: int, page_size: int) -> None:
        """``proj`` [T, ...]: q heads in the columns [0, H D), k heads from ``k_off``, value rows from ``v_off``.  Every q
        and k head has its dimensions (2i, 2i + 1), i < rot_dims / 2, turned by position * freq[i] (32-bit); q in place,
        k into ``k_cache`` and the value rows into ``v_cache`` at ``slots`` (None: nothing is cached)."""
        self._check(self.lib.ts_rope_pairs_write(_ptr(proj), proj.stride(0), k_off, v_off, _ptr(positions), _ptr(freq),
                                                 float(magnitude), int(rot_dims), _ptr(k_cache), _ptr(v_cache), _ptr(slots),
                                                 proj.shape[0], H, G, D, V, page_size, _code(proj.dtype), self._stream()),
                    "rope_pairs_write")

    # -- routed feed-forward ---------------------------------------------------------------------------------
    def router_topk(self, idx, weights, x, w_router, softmax: bool, renormalize: bool, correction=None) -> None:
        """idx (int32 [T, top]), weights (float32 [T, top]): the ``top`` experts with the largest router
        logits w_router (float32 [E, K]) . x, and their scores (sigmoid, or softmax over all experts).  With
        ``correction`` (float32 [E]) the choice goes by score + correction; the weights stay the scores."""
        T, top = idx.shape
        E, K = w_router.shape
        self._check(self.lib.ts_router_topk(_ptr(idx), _ptr(weights), _ptr(x), _ptr(w_router), T, E, K, top,
                                            1 if softmax else 0, 1 if renormalize else 0, _code(x.dtype), _ptr(correction),
                                            self._stream()), "router_topk")

    def moe_align(self, idx, E: int, with_tiles: int | None = None):
        """Sorts the (token, choice) pairs of ``idx`` by expert on the device.  Returns (offsets [E + 1],
        order [P], place [P], tiles): work buffers of this object, valid until the next call.  ``with_tiles``:
        only the experts below it get row tiles for the grouped products (the others have no weights)."""
        P = idx.numel()
        dev = idx.device
        rows = self.lib.ts_moe_tile_rows()
        offsets = self._buffer("moe_offsets", E + 1, torch.int32, dev, floor=1024)
        order = self._buffer("moe_order", P, torch.int32, dev, floor=1 << 14)
        place = self._buffer("moe_place", P, torch.int32, dev, floor=1 << 14)
        tiles = self._buffer("moe_tiles", 1 + 2 * (-(-P // rows) + E), torch.int32, dev, floor=1 << 12)
        self._check(self.lib.ts_moe_align(_ptr(idx), P, E, _ptr(offsets), _ptr(order), _ptr(place), _ptr(tiles),
                                          E if with_tiles is None else int(with_tiles), self._stream()), "moe_align")
        return offsets, order, place, tiles

    def grouped_linear(self, out, x, w, order, row_scale, offsets, tiles, top: int, act: str = "none") -> None:
        """out[i] = act(a_i . w[e_i]^T) for the P sorted places i (``w`` [E, N, K]); a_i = x[i], or with
        ``order``: x[order[i] // top] (times row_scale[order[i]], rounded to x's type)."""
        P, N = out.shape
        E, _, K = w.shape
        self._check(self.lib.ts_grouped_linear(_ptr(out), _ptr(x), _ptr(w), _ptr(order), _ptr(row_scale), _ptr(offsets),
                                               _ptr(tiles), P, E, top, N, K, self.ACTIVATIONS[act], _code(x.dtype),
                                               _code(out.dtype), self._stream()), "grouped_linear")

    def moe_gather(self, xs, x, order, row_scale, top: int) -> None:
        """xs[i] = x[order[i] // top] (times row_scale[order[i]], rounded to x's type): the experts' input rows
        in sorted order."""
        P, K = xs.shape
        self._check(self.lib.ts_moe_gather(_ptr(xs), _ptr(x), _ptr(order), _ptr(row_scale), P, top, K, _code(x.dtype),
                                           self._stream()), "moe_gather")

    def moe_combine(self, out, y, place, pair_weights, top: int, x=None, pass_from=None, add=None) -> None:
        """out[t] = sum over a token's choices r of (pair_weights[t, r] *) y[place[t top + r]] (y float32).  With ``x``
        ([T, N], out's type) and ``pass_from`` (one int32 on the device): a pair sorted to that place or a later
        one adds x[t] instead of a row of y (experts that return their input).  ``add`` ([T, N], out's type): added
        to every token's sum (the output of an expert that every token uses)."""
        T, N = out.shape
        self._check(self.lib.ts_moe_combine(_ptr(out), _ptr(y), _ptr(place), _ptr(pair_weights), T, top, N,
                                            _code(out.dtype), _ptr(x), _ptr(pass_from), _ptr(add), self._stream()),
                    "moe_combine")

    PAIR_PLAIN, PAIR_GATED = 0, 1
    # The many-row products whose epilogue saves a kernel (gate/up with the activation, q/k/v with rotation and
    # cache write) run on this library's kernel for pairs of SMs where its schedule is the shorter one; 0: never.
    # ("gated": the gate/up product only)
    pair_gemm = os.environ.get("TURINGSERVE_B200_PAIR_GEMM", "1") != "0"
    pair_qkv = os.environ.get("TURINGSERVE_B200_PAIR_GEMM", "1") not in ("0", "gated")

    def pair_wins(self, M: int, N: int, K: int, saved_bytes: float) -> bool:
        """Whether the pair kernel's schedule (rounds of 256 x 256 tiles over the pairs of SMs, 0.42 us a
        64-wide k-block: 79 us measured for 2,048 x 17,920 x 1,536, 353 us for 2,048 x 37,888 x 3,584) is shorter
        than the library product at 1.35 PFLOP/s followed by a kernel that moves ``saved_bytes`` at 5.5 TB/s
        (2,048 tokens of the 1.5B shape: 80 + 19 us; 544 tokens of the 14B shape: 113 + 9 us against 147)."""
        if not (self.pair_gemm and self.gemm_mode in ("auto", "tc")):
            return False
        tiles = -(-M // 256) * -(-N // 256)
        rounds = -(-tiles // max(1, self.num_sms // 2))
        pair_us = rounds * -(-K // 64) * 0.42 + 3.0
        library_us = 2.0 * M * N * K / 1.35e9 + 3.0 + saved_bytes / 5.5e6 + 2.0
        return pair_us < library_us

    def linear_pair(self, out, x, w, bias, epilogue: int) -> bool:
        """The many-row bfloat16 product on pairs of SMs.  ``epilogue`` PAIR_PLAIN: out[M, N] = x @ w^T + bias;
        PAIR_GATED: out[M, N / 2] = silu(g) * u, the rows of ``w`` in blocks of 64 gates and their 64 ups.
        False when the kernel does not take the shape."""
        M, K = x.shape
        N = w.shape[0]
        rc = self.lib.ts_linear_pair(_ptr(out), _ptr(x), _ptr(w), _ptr(bias), M, N, K, epilogue, self._stream())
        if rc == self.UNSUPPORTED:
            return False
        self._check(rc, "linear_pair")
        return True

    def partial_scratch(self, floats: int, device) -> torch.Tensor:
        """The buffer deferred products leave their partial sums in (one deferred product at a time)."""
        return self._buffer("partials", floats, torch.float32, device, floor=1 << 20)

    def tc_splits(self, M: int, N: int, K: int) -> int:
        """Pieces K is cut into for a few-token product, so that about one tile lands on every SM."""
        if M > 128:
            return 1
        tiles = -(-N // 128)
        k_blocks = -(-K // 64)
        if tiles >= self.num_sms // 2:
            return 1
        # partial sums cost 8*M*N bytes per split (written, read back): keep that below the weights' 2*N*K
        traffic_cap = max(1, K // (4 * M))
        # every split is one more partial sum for the consuming kernel to fetch: at least four k-blocks
        # a split, ten splits at most (measured on the 1.5B shape at 8 tokens: 1.555 -> 1.501 ms a step
        # against twelve splits everywhere)
        return max(1, min(self.num_sms // tiles, max(2, k_blocks // 4), traffic_cap, self.max_splits))

    def tc_status(self) -> int:
        """0 when no tensor-core block (GEMM or attention) ever gave up on a wait (synchronises the device)."""
        return (int(self.lib.ts_linear_tc_status()) or int(self.lib.ts_attention_prefill_tc_status())
                or int(self.lib.ts_attention_decode_tma_status()) or int(self.lib.ts_decode_step_status()))

    STATUS_WORDS = 4            # what ts_sample* report beside the tokens: GEMM, prompt attention, TMA decode attention, fused decode step

    def fault_reported(self, status) -> str:
        """The engine found non-zero status words beside a step's tokens: a block of one of the
        kernels with bounded waits gave up, so the step's output cannot be trusted.  Takes the kernel
        concerned off the product path (its slower counterpart runs from the next step on), clears
        the words, and says what happened."""
        names = ("tensor-core product", "tensor-core prompt attention", "TMA decode attention", "fused decode step")
        hit = [f"{names[i]} (wait {int(v)})" for i, v in enumerate(status) if int(v)]
        if int(status[0]):
            self.gemm_mode = "library"
        if int(status[1]):
            self.use_tc_attention = False
        if int(status[2]):
            self.decode_kernel = "cp"
        if int(status[3]):
            self.use_fused_step = False
        self.lib.ts_clear_status(self._stream())
        return "a kernel gave up on a bounded wait: " + ", ".join(hit) + "; its fallback runs from now on"

    def feed_tokens(self, ids, rows, src, tokens, vocab: int) -> None:
        """ids[rows[i]] = tokens[src[i]] on the device (all int32)."""
        self._check(self.lib.ts_feed_tokens(_ptr(ids), _ptr(rows), _ptr(src), _ptr(tokens), rows.shape[0], vocab,
                                            self._stream()), "feed_tokens")

    def sample(self, out, logits, fparams, iparams, status_out=None) -> None:
        """``status_out``: STATUS_WORDS int32 that receive the kernels' status words (see fault_reported)."""
        S, V = logits.shape
        self._check(self.lib.ts_sample(_ptr(out), _ptr(logits), _ptr(fparams), _ptr(iparams), S, V,
                                       _ptr(status_out), self._stream()), "sample")

    def sample_greedy(self, out, logits, status_out=None) -> None:
        """Every row greedy: the draw without parameters, each row spread over many blocks."""
        S, V = logits.shape
        need = 2 * S * self.lib.ts_sample_greedy_parts(V)
        scratch = self._buffer("greedy_scratch", need, torch.int32, logits.device, floor=2 * 256 * 64)
        counters = self._buffer("greedy_counters", S, torch.int32, logits.device, floor=1024, zero=True)
        self._check(self.lib.ts_sample_greedy(_ptr(out), _ptr(logits), S, V, _ptr(scratch), _ptr(counters),
                                              _ptr(status_out), self._stream()), "sample_greedy")

    def penalize(self, logits, ids, meta, pen) -> None:
        S, V = logits.shape
        self._check(self.lib.ts_penalize(_ptr(logits), _ptr(ids), _ptr(meta), _ptr(pen), S, V,
                                         self._stream()), "penalize")


def ops():
    """The kernel object; builds and loads the CUDA library on first use.  Raises when there is
    no CUDA device or the library cannot be built: there is no fallback."""
    global _OPS
    if _OPS is None:
        if not torch.cuda.is_available():
            raise KernelError("turingserve_b200 needs a CUDA device (sm_100a); none is available")
        _OPS = CudaOps(build())
    return _OPS


def use(ops_object) -> None:
    """Install another object behind ``ops()`` (tests drive the engine's host logic with a plain
    torch twin of every kernel this way); ``use(None)`` goes back to the CUDA library."""
    global _OPS
    _OPS = ops_object


__all__ = ["CudaOps", "Deferred", "KernelError", "LazyProduct", "build", "library_path", "ops", "use"]
