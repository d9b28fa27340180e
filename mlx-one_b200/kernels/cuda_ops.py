"""The kernel set of the engine: thin Python wrappers around the C launchers.

Each method allocates its output with torch, checks dtypes and shapes, and passes raw
pointers and the current CUDA stream to the library. There is no fallback: constructing
``CudaOps`` fails if the library cannot be built or loaded or no CUDA device is present.

Matrix products in bfloat16 go through ``torch.matmul`` (cuBLAS), as the reference uses its
library's matrix product (nn.Linear, src/mlx_one/models/language/lfm2/reference_math.py:33-34);
in float32 they go through this library's own FMA kernel, which never uses a
reduced-precision mode.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch

from ..parts.base import NormedInput
from .build import KernelBuildError, library_path

_F32, _BF16 = 0, 1
_c_int, _c_float, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong


class KernelError(RuntimeError):
    """A kernel launcher refused its arguments or a kernel reported a fault."""


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels exist for float32 and bfloat16, not {dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


class CudaOps:
    name = "cuda"

    def __init__(self, device: torch.device | str = "cuda:0", verbose: bool = True) -> None:
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelBuildError("the engine needs a CUDA device (sm_100a); it has no CPU path")
        try:
            self.lib = ctypes.CDLL(str(library_path(verbose=verbose)))
        except OSError as exc:
            raise KernelBuildError(f"cannot load the CUDA extension: {exc}") from exc
        self.lib.mlxone_last_error.restype = ctypes.c_char_p
        self.lib.mlxone_gated_delta_scratch.restype = ctypes.c_longlong
        self.lib.mlxone_gated_delta_state.restype = ctypes.c_longlong
        self.lib.mlxone_lightning_scratch.restype = ctypes.c_longlong
        self.lib.mlxone_state_space_scratch.restype = ctypes.c_longlong
        if self.lib.mlxone_abi_version() != 1:
            raise KernelBuildError("the CUDA extension is of another version; rebuild it")
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0
        self.tensor_core_attention = True
        self.skinny_products = True
        # A norm applied inside the product that consumes it (the skinny product reads the 32-bit
        # rows, all warps sharing the sums of squares, the norm's weights staged before the wait
        # for the kernel before it): no norm kernel, but every block reads rows of twice the size.
        # Decode steps of the 1.2B shape at 4096 keys: batch 1 / 2 / 4 / 6 0.578 / 0.588 / 0.615 /
        # 0.644 ms against 0.597 / 0.610 / 0.642 / 0.660 ms with the norm kernel; batch 8 0.68
        # against 0.67 ms, batch 16 0.95 against 0.89 ms. So up to `fused_norm_max_rows` rows.
        self.fused_norms = True
        self.fused_norm_max_rows = 6
        self.tcgen05_min_rows = 128
        self.tcgen05_attention = True     # prefill attention with tcgen05 where it takes the geometry
        # ... and with the keys of its few items cut into parts when a launch has fewer items than SMs
        self.prefill_key_splits = True
        # decode attention: key splits merged by a thread-block cluster through distributed shared
        # memory instead of a scratch buffer and a merge kernel (one launch fewer a layer), for up
        # to `cluster_merge_max_splits` splits. Measured inside the decode step of the 1.2B shape at
        # 4096 keys (the kernel before attention is the qkv product, whose blocks still hold their
        # SMs' shared memory when the clusters are placed): clusters of 2 and 3 (batch 20 to 32)
        # 1.004 against 1.036 ms and 1.08 against 1.12 ms; clusters of 8 at batch 8 take either
        # 19.5 or 31 us a launch where nine splits and the merge kernel take 17.5 + 3 us
        # (0.686 against 0.667 ms a step); clusters of 4 at batch 12 (16 rows, four of them
        # fillers) 37 against 23.6 us a launch, at batch 16 29 against 30 us.
        self.cluster_merge = True
        self.cluster_merge_max_splits = 3
        # a step of single tokens: q/k norm, rotation and the page write inside the decode
        # attention kernel instead of a kernel of their own before it
        self.fused_decode_attention = True
        # a mixed step's leading single-token requests go to the decode attention kernel when
        # there are at least this many of them
        self.split_singles_from = 1
        self.tcgen05_always = False       # tests: take the tcgen05 kernel whenever it can run
        self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        # tcgen05 products (TMA + tensor memory) for more rows than the skinny kernel takes
        self.tcgen05_products = bool(self.lib.mlxone_gemm_tcgen05_available())
        # 33 to 128 rows: a tcgen05 product with swapped operands (weights as the 128-row operand,
        # K split over a thread-block cluster). Off: at 64 rows only w2 is faster than the library's
        # product (12.0 us against 13.3 us; in_proj 10.7 us against 6.9 us, w13 + SwiGLU 21.7 us
        # against 17.3 us), because a block's start and epilogue (about 8 us) are not hidden
        self.swapped_products = False
        self._swapped_rows = self.lib.mlxone_gemm_tcgen05_swapped_max_rows()
        self._skinny_rows = self.lib.mlxone_gemm_skinny_max_rows()
        # The skinny kernel takes up to 32 rows, but beyond 8 (more than one group of eight
        # tokens per tensor-core instruction) the library's product is faster: a decode step at
        # batch 16 takes 0.91 ms against 1.07 ms, at batch 32 0.98 ms against 1.91 ms
        self.skinny_max_rows = 8
        # With an epilogue of its own (SwiGLU, the residual add, the conv update) it is the faster
        # one up to 16 rows: out_proj 4.3 us against 5.7 us, w2 10.5 us against 13.0 us, w13 with
        # its gate 14.6 us against 12.9 us plus a gate kernel
        self.skinny_fused_max_rows = 16
        self._sample_scratch: torch.Tensor | None = None
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()

    # ------------------------------------------------------------------ plumbing

    def _stream(self) -> int:
        """The current stream's handle (the capture stream while a graph is captured). torch's
        raw query costs a fraction of building a Stream object, which a step would pay a
        hundred times."""
        if _raw_stream is not None:
            return _raw_stream(self._device_index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def _call(self, name: str, *args: Any) -> None:
        code = getattr(self.lib, name)(*args, _c_void_p(self._stream()))
        if code != 0:
            raise KernelError(self.lib.mlxone_last_error().decode())
        self.launches += 1

    def _need_rows(self, tensor: torch.Tensor, dtype: torch.dtype, what: str) -> None:
        """Rows whose values lie together; the rows themselves may be a slice of a wider matrix."""
        if (tensor.dtype != dtype or tensor.dim() != 2 or tensor.stride(1) != 1
                or tensor.device != self.device):
            raise KernelError(f"{what} must be {dtype} rows on {self.device}, got {tensor.dtype} "
                              f"{tuple(tensor.shape)} with strides {tensor.stride()} on {tensor.device}")

    def _need(self, tensor: torch.Tensor, dtype: torch.dtype, what: str) -> None:
        if tensor.dtype != dtype or not tensor.is_contiguous() or tensor.device != self.device:
            raise KernelError(f"{what} must be a contiguous {dtype} tensor on {self.device}, got "
                              f"{tensor.dtype} {tuple(tensor.shape)} on {tensor.device}")

    def set_dependent_launches(self, enabled: bool) -> None:
        """Programmatic dependent launches on the decode path: a kernel may start, and fetch
        its weights, while the one before it finishes."""
        self.lib.mlxone_set_pdl(1 if enabled else 0)

    ERRORS = {1: "a token id outside the vocabulary",
              2: "a key written to a position that has no page",
              3: "a key read from a position that has no page",
              9: "a wait inside a tcgen05 kernel that gave up"}

    def describe_error(self, code: int) -> KernelError:
        return KernelError(f"a kernel reported {self.ERRORS.get(code, f'code {code}')}")

    def check_errors(self) -> None:
        """Reads the device error flag (synchronises) and raises if a kernel set it."""
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            raise self.describe_error(code)

    # ------------------------------------------------------------------ size checks

    def check_attention_sizes(self, heads: int, kv_heads: int, head_dim: int) -> None:
        if heads % kv_heads:
            raise KernelError(f"{heads} query heads cannot share {kv_heads} key heads")
        if not 2 <= head_dim <= 1024:
            raise KernelError(f"head size {head_dim} is outside 2..1024")

    # ------------------------------------------------------------------ ops

    def embedding(self, ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        self._need(ids, torch.int32, "token ids")
        out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=self.device)
        self._call("mlxone_embedding", _c_void_p(_ptr(ids)), _c_void_p(_ptr(table)),
                   _c_void_p(_ptr(out)), _c_int(ids.numel()), _c_int(table.shape[1]),
                   _c_int(table.shape[0]), _c_int(_dtype_code(table.dtype)),
                   _c_void_p(_ptr(self.error_flag)))
        return out

    def add_rmsnorm(self, residual, delta, weight, eps, dtype, delta_scale=1.0):
        self._need(residual, torch.float32, "residual")
        self._need(weight, torch.float32, "norm weight")
        if delta is not None:
            self._need(delta, dtype, "delta")
            if delta.shape != residual.shape:
                raise KernelError("delta and residual differ in shape")
        rows, hidden = residual.shape
        if weight.numel() != hidden:
            raise KernelError(f"norm weight has {weight.numel()} entries, rows have {hidden}")
        out = torch.empty((rows, hidden), dtype=dtype, device=self.device)
        self._call("mlxone_add_rmsnorm", _c_void_p(_ptr(residual)), _c_void_p(_ptr(delta)),
                   _c_void_p(_ptr(weight)), _c_void_p(_ptr(out)), _c_int(rows), _c_int(hidden),
                   _c_float(eps), _c_int(_dtype_code(dtype)), _c_float(delta_scale))
        return out

    def gather_rows(self, residual, delta, rows):
        self._need(residual, torch.float32, "residual")
        self._need(rows, torch.int32, "rows")
        count, hidden = rows.numel(), residual.shape[1]
        picked = torch.empty((count, hidden), dtype=torch.float32, device=self.device)
        picked_delta = None
        code = _F32
        if delta is not None:
            picked_delta = torch.empty((count, hidden), dtype=delta.dtype, device=self.device)
            code = _dtype_code(delta.dtype)
        self._call("mlxone_gather_rows", _c_void_p(_ptr(residual)), _c_void_p(_ptr(delta)),
                   _c_void_p(_ptr(rows)), _c_void_p(_ptr(picked)), _c_void_p(_ptr(picked_delta)),
                   _c_int(count), _c_int(hidden), _c_int(residual.shape[0]), _c_int(code))
        return picked, picked_delta

    # epilogues of the skinny product
    _STORE, _SWIGLU, _ADD, _STORE_F32 = 0, 1, 2, 3
    _ACTIVATE = 16          # + the activation's code: a bfloat16 store of the activated product
    _GATED = 32             # + the activation's code: as _SWIGLU with that gate

    def _skinny(self, a, w, fused=False) -> bool:
        """Whether a[M, K] @ w[N, K]^T goes to the weight-streaming kernel: bfloat16, few rows,
        16-byte aligned rows. Everything else goes to the library product. ``fused``: the
        product has an epilogue that the library's product would need another kernel for."""
        most = max(self.skinny_max_rows, self.skinny_fused_max_rows) if fused else self.skinny_max_rows
        return (self.skinny_products and a.dtype == torch.bfloat16
                and 0 < a.shape[0] <= min(self._skinny_rows, most)
                and a.shape[1] % 8 == 0
                and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def enable_tcgen05(self, enabled: bool = True) -> bool:
        """Routes bfloat16 products with more rows than the skinny kernel takes to the
        tcgen05 kernel (TMA loads, accumulator in tensor memory) instead of the library."""
        self.tcgen05_products = bool(enabled) and bool(self.lib.mlxone_gemm_tcgen05_available())
        if not self.tcgen05_products:
            self.swapped_products = False
        return self.tcgen05_products

    def _tcgen05(self, a, w, epilogue=0) -> bool:
        """Whether a[M, K] @ w[N, K]^T goes to the tcgen05 kernel. It needs 16-byte aligned
        rows and at least 128 rows (its tiles are 128 x 256 and each persistent block walks
        whole tiles), and it is chosen where it is faster than the library's product plus the
        kernel that the library's product then needs: with the fused SwiGLU epilogue, which
        saves a pass over the widest activation (2048 rows: 100 us against 153 us; 512 rows: 35
        against 41), when its tiles fill the SMs to 60 %. Plain products and products added into
        the residual stream go to the library, which is faster at every row count measured
        (2048 rows: in_proj 37.7 us against 45.3, qkv 20.7 against 30.8, out_proj 14.8 against
        24.8 with the residual epilogue, w2 47 against 62; 8192 rows: 142 / 73 / 49 / 181 us
        against 156 / 82 / 77 / 244); their result is added by the next norm kernel."""
        if not (self.tcgen05_products and a.dtype == torch.bfloat16
                and a.shape[0] >= self.tcgen05_min_rows
                and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1
                and w.is_contiguous() and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            return False
        if self.tcgen05_always:
            return True
        if epilogue != self._SWIGLU:
            return False
        tiles = -(-a.shape[0] // 128) * -(-(w.shape[0] // 2) // 128)
        evenness = tiles / (-(-tiles // self._sm_count) * self._sm_count)
        return evenness >= 0.6

    def _tcgen05_call(self, a, w, bias, out, ldo, epilogue) -> None:
        self._call("mlxone_gemm_tcgen05", _c_void_p(_ptr(a)), _c_int(a.stride(0)),
                   _c_void_p(_ptr(w)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(out)), _c_int(ldo),
                   _c_int(a.shape[0]), _c_int(w.shape[0]), _c_int(a.shape[1]), _c_int(epilogue),
                   _c_void_p(_ptr(self.error_flag)))

    def _swapped(self, a, w) -> bool:
        """Whether a[M, K] @ w[N, K]^T goes to the tcgen05 product with swapped operands: more
        rows than the skinny kernel takes, at most 128, 16-byte aligned rows."""
        return (self.swapped_products and a.dtype == torch.bfloat16
                and min(self._skinny_rows, self.skinny_max_rows) < a.shape[0] <= self._swapped_rows
                and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1
                and w.is_contiguous() and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def _swapped_call(self, a, w, bias, out, ldo, epilogue) -> None:
        self._call("mlxone_gemm_tcgen05_swapped", _c_void_p(_ptr(a)), _c_int(a.stride(0)),
                   _c_void_p(_ptr(w)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(out)), _c_int(ldo),
                   _c_int(a.shape[0]), _c_int(w.shape[0]), _c_int(a.shape[1]), _c_int(epilogue),
                   _c_void_p(_ptr(self.error_flag)))

    def _skinny_call(self, a, w, bias, out, ldo, epilogue) -> None:
        self._call("mlxone_gemm_skinny", _c_void_p(_ptr(a)), _c_int(a.stride(0)),
                   _c_void_p(_ptr(w)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(out)), _c_int(ldo),
                   _c_int(a.shape[0]), _c_int(w.shape[0]), _c_int(a.shape[1]), _c_int(epilogue))

    def _check_product(self, a, w) -> None:
        if a.dtype != w.dtype:
            raise KernelError(f"matrix product of {a.dtype} with {w.dtype}")
        if a.dim() != 2 or w.dim() != 2 or w.shape[1] != a.shape[1]:
            raise KernelError(f"matrix product of {tuple(a.shape)} with {tuple(w.shape)}^T")

    # ---- norms applied inside the product that consumes them

    def can_fuse_norm(self, residual, dtype) -> bool:
        """Whether RMSNorm(residual) can be applied by the skinny product while it loads its
        input (bfloat16, up to 16 rows, the rows fit into shared memory)."""
        return (self.fused_norms and self.skinny_products and dtype == torch.bfloat16
                and residual.shape[0] <= self.fused_norm_max_rows
                and residual.dtype == torch.float32 and residual.is_contiguous()
                and bool(self.lib.mlxone_gemm_skinny_norm_fits(residual.shape[0], residual.shape[1])))

    def _normed_call(self, a, w, bias, out, ldo, epilogue) -> None:
        self._need(w, torch.bfloat16, "w")
        if w.shape[1] != a.residual.shape[1]:
            raise KernelError(f"matrix product of {tuple(a.shape)} with {tuple(w.shape)}^T")
        self._call("mlxone_gemm_skinny_norm", _c_void_p(_ptr(a.residual)),
                   _c_int(a.residual.stride(0)), _c_void_p(_ptr(a.weight)), _c_float(a.eps),
                   _c_void_p(_ptr(w)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(out)), _c_int(ldo),
                   _c_int(a.shape[0]), _c_int(w.shape[0]), _c_int(a.shape[1]), _c_int(epilogue))

    def linear(self, a, w, bias=None, out_dtype=None):
        """a[M, K] @ w[N, K]^T (+ bias[N], float32). ``out_dtype``: a's dtype, or float32."""
        if isinstance(a, NormedInput):
            out_dtype = out_dtype or a.dtype
            out = torch.empty((a.shape[0], w.shape[0]), dtype=out_dtype, device=self.device)
            self._normed_call(a, w, bias, out, w.shape[0],
                              self._STORE_F32 if out_dtype == torch.float32 else self._STORE)
            return out
        self._check_product(a, w)
        out_dtype = out_dtype or a.dtype
        m, k = a.shape
        n = w.shape[0]
        if a.dtype == torch.float32:
            self._need(a, torch.float32, "a")
            self._need(w, torch.float32, "w")
            out = torch.empty((m, n), dtype=torch.float32, device=self.device)
            self._call("mlxone_gemm_f32", _c_void_p(_ptr(a)), _c_int(k), _c_void_p(_ptr(w)),
                       _c_int(k), _c_void_p(_ptr(bias)), _c_void_p(_ptr(out)), _c_int(n),
                       _c_int(m), _c_int(n), _c_int(k))
            return out
        if self._skinny(a, w):
            out = torch.empty((m, n), dtype=out_dtype, device=self.device)
            self._skinny_call(a, w, bias, out, n,
                              self._STORE_F32 if out_dtype == torch.float32 else self._STORE)
            return out
        if self._swapped(a, w):
            out = torch.empty((m, n), dtype=out_dtype, device=self.device)
            self._swapped_call(a, w, bias, out, n,
                               self._STORE_F32 if out_dtype == torch.float32 else self._STORE)
            return out
        if self._tcgen05(a, w, self._STORE):
            out = torch.empty((m, n), dtype=out_dtype, device=self.device)
            self._tcgen05_call(a, w, bias, out, n,
                               self._STORE_F32 if out_dtype == torch.float32 else self._STORE)
            return out
        if out_dtype == torch.float32:
            out = torch.mm(a, w.t(), out_dtype=torch.float32)
        else:
            out = torch.mm(a, w.t())
        if bias is not None:
            self._call("mlxone_add_bias", _c_void_p(_ptr(out)), _c_void_p(_ptr(bias)), _c_int(m),
                       _c_int(n), _c_int(_dtype_code(out.dtype)))
        return out

    def linear_swiglu(self, a, gate_up):
        """silu(a @ gate^T) * (a @ up^T) with gate_up = [gate rows; up rows]: one kernel for
        few rows, else a product followed by the gate kernel."""
        if isinstance(a, NormedInput):
            width = gate_up.shape[0] // 2
            out = torch.empty((a.shape[0], width), dtype=a.dtype, device=self.device)
            self._normed_call(a, gate_up, None, out, width, self._SWIGLU)
            return out
        self._check_product(a, gate_up)
        if self._skinny(a, gate_up, fused=True):
            width = gate_up.shape[0] // 2
            out = torch.empty((a.shape[0], width), dtype=a.dtype, device=self.device)
            self._skinny_call(a, gate_up, None, out, width, self._SWIGLU)
            return out
        if self._swapped(a, gate_up):
            width = gate_up.shape[0] // 2
            out = torch.empty((a.shape[0], width), dtype=a.dtype, device=self.device)
            self._swapped_call(a, gate_up, None, out, width, self._SWIGLU)
            return out
        if self._tcgen05(a, gate_up, self._SWIGLU):
            width = gate_up.shape[0] // 2
            out = torch.empty((a.shape[0], width), dtype=a.dtype, device=self.device)
            self._tcgen05_call(a, gate_up, None, out, width, self._SWIGLU)
            return out
        return self.swiglu(self.linear(a, gate_up))

    def linear_add(self, a, w, bias, residual, scale=1.0):
        """Adds scale * (a @ w^T (+ bias)) to the float32 ``residual``. Returns None if it was
        added in place (few rows: the product's epilogue does it), else the product, which the
        caller adds, with its factor, with the next norm."""
        self._check_product(a, w)
        if self._skinny(a, w, fused=True):
            self._need(residual, torch.float32, "residual")
            if scale == 1.0:
                self._skinny_call(a, w, bias, residual, residual.shape[1], self._ADD)
            else:
                self._call("mlxone_gemm_skinny_scaled_add", _c_void_p(_ptr(a)), _c_int(a.stride(0)),
                           _c_void_p(_ptr(w)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(residual)),
                           _c_int(residual.shape[1]), _c_int(a.shape[0]), _c_int(w.shape[0]),
                           _c_int(a.shape[1]), _c_float(scale))
            return None
        if scale != 1.0:
            return self.linear(a, w, bias)
        if self._swapped(a, w):
            self._need(residual, torch.float32, "residual")
            self._swapped_call(a, w, bias, residual, residual.shape[1], self._ADD)
            return None
        if self._tcgen05(a, w, self._ADD):
            self._need(residual, torch.float32, "residual")
            self._tcgen05_call(a, w, bias, residual, residual.shape[1], self._ADD)
            return None
        return self.linear(a, w, bias)

    def linear_gated(self, a, gate_up, kind):
        """act(a @ gate^T) * (a @ up^T) with gate_up = [gate rows; up rows], for the activations
        of ``ACTIVATIONS``: silu takes the fused kernels of ``linear_swiglu``; for the others the
        gate is the skinny product's epilogue for few rows (also with the norm of its input
        applied while loading), else the product and one kernel for the gate."""
        if kind == "silu":
            return self.linear_swiglu(a, gate_up)
        if kind not in self.ACTIVATIONS:
            raise KernelError(f"unknown activation {kind!r}")
        epilogue = self._GATED + self.ACTIVATIONS[kind]
        width = gate_up.shape[0] // 2
        if isinstance(a, NormedInput):
            out = torch.empty((a.shape[0], width), dtype=a.dtype, device=self.device)
            self._normed_call(a, gate_up, None, out, width, epilogue)
            return out
        self._check_product(a, gate_up)
        if self._skinny(a, gate_up, fused=True):
            out = torch.empty((a.shape[0], width), dtype=a.dtype, device=self.device)
            self._skinny_call(a, gate_up, None, out, width, epilogue)
            return out
        both = self.linear(a, gate_up)
        rows, twice = both.shape
        out = torch.empty((rows, twice // 2), dtype=both.dtype, device=self.device)
        self._call("mlxone_gated_activation", _c_void_p(_ptr(both)), _c_void_p(_ptr(out)),
                   _c_int(rows), _c_int(twice // 2), _c_int(self.ACTIVATIONS[kind]),
                   _c_int(_dtype_code(both.dtype)))
        return out

    # ---- activations of a feed-forward without a gate

    ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "relu": 3, "xielu": 4}

    def activation(self, x, kind, params=None):
        """relu2 (max(z, 0)^2), gelu_tanh, silu, relu or xielu of every value. ``params``: the
        two numbers (a, b) of xielu: a z^2 + z / 2 above zero, b (e^z - 1 - z) + z / 2 below."""
        if kind not in self.ACTIVATIONS:
            raise KernelError(f"unknown activation {kind!r}")
        if (kind == "xielu") != (params is not None):
            raise KernelError("xielu, and only xielu, takes two numbers")
        self._need(x, x.dtype, "x")
        out = torch.empty_like(x)
        a, b = params or (0.0, 0.0)
        self._call("mlxone_activation_shaped", _c_void_p(_ptr(x)), _c_void_p(_ptr(out)),
                   _c_ll(x.numel()), _c_int(self.ACTIVATIONS[kind]), _c_float(a), _c_float(b),
                   _c_int(_dtype_code(x.dtype)))
        return out

    def linear_act(self, a, w, kind, params=None):
        """act(a @ w^T): for few rows the activation is the skinny product's epilogue (also with
        the norm of its input applied while loading); else the product, then the activation
        kernel. ``params``: the two numbers of an activation that has some (xielu)."""
        if kind not in self.ACTIVATIONS:
            raise KernelError(f"unknown activation {kind!r}")
        if params is not None:
            if isinstance(a, NormedInput):
                a = a.materialize()
            self._check_product(a, w)
            if self._skinny(a, w, fused=True):
                out = torch.empty((a.shape[0], w.shape[0]), dtype=a.dtype, device=self.device)
                self._call("mlxone_gemm_skinny_shaped", _c_void_p(_ptr(a)), _c_int(a.stride(0)),
                           _c_void_p(_ptr(w)), _c_void_p(None), _c_void_p(_ptr(out)),
                           _c_int(w.shape[0]), _c_int(a.shape[0]), _c_int(w.shape[0]),
                           _c_int(a.shape[1]), _c_int(self.ACTIVATIONS[kind]),
                           _c_float(params[0]), _c_float(params[1]))
                return out
            return self.activation(self.linear(a, w), kind, params)
        epilogue = self._ACTIVATE + self.ACTIVATIONS[kind]
        if isinstance(a, NormedInput):
            out = torch.empty((a.shape[0], w.shape[0]), dtype=a.dtype, device=self.device)
            self._normed_call(a, w, None, out, w.shape[0], epilogue)
            return out
        self._check_product(a, w)
        if self._skinny(a, w, fused=True):
            out = torch.empty((a.shape[0], w.shape[0]), dtype=a.dtype, device=self.device)
            self._skinny_call(a, w, None, out, w.shape[0], epilogue)
            return out
        return self.activation(self.linear(a, w), kind)

    # ---- the stream's first value, the streams kept over the layers, convolutions over time

    def embedding_pairs(self, ids, table, scale, pairs, *, rule, ctx, view, out=None):
        """float32 [tokens, hidden]: the table's row times ``scale``, plus (with ``pairs``) the
        row of the second table that the token and the one before it in its request choose;
        ``view`` is the int32 slot per request that holds the last token seen plus one."""
        self._need(ids, torch.int32, "token ids")
        tokens, hidden = ids.numel(), table.shape[1]
        if out is None:
            out = torch.empty((tokens, hidden), dtype=torch.float32, device=self.device)
        self._need(out, torch.float32, "out")
        self._need(table, table.dtype, "table")
        buckets = mul_prev = mul_cur = 0
        state = slots = None
        if pairs is not None:
            self._need(pairs, table.dtype, "pairs")
            buckets, mul_prev, mul_cur = rule
            if pairs.shape != (buckets + 1, hidden):
                raise KernelError("the pair table has one row per bucket and one more")
            self._need(view.state, torch.int32, "state")
            state, slots = view.state, view.slots
        self._call("mlxone_embedding_pairs", _c_void_p(_ptr(ids)), _c_void_p(_ptr(table)),
                   _c_float(scale), _c_void_p(_ptr(pairs)), _c_int(buckets), _c_ll(mul_prev),
                   _c_ll(mul_cur), _c_void_p(_ptr(ctx.token_request)),
                   _c_void_p(_ptr(ctx.request_start)), _c_void_p(_ptr(state)),
                   _c_void_p(_ptr(slots)), _c_void_p(_ptr(out)), _c_int(tokens), _c_int(hidden),
                   _c_int(table.shape[0]), _c_int(_dtype_code(table.dtype)),
                   _c_void_p(_ptr(self.error_flag)))
        return out

    def stream_average(self, kept, weights, count, out):
        """out = sum_j weights[j] * kept[j], j < count (32-bit, added in that order); without
        weights a copy of kept[0]. ``out`` may be a stream of ``kept`` beyond ``count``."""
        self._need(kept, torch.float32, "kept")
        self._need(out, torch.float32, "out")
        if weights is not None:
            self._need(weights, torch.float32, "weights")
            if weights.numel() < count or kept.shape[0] < count:
                raise KernelError(f"{count} streams are averaged, fewer are given")
        self._call("mlxone_stream_average", _c_void_p(_ptr(kept)), _c_ll(kept.stride(0)),
                   _c_void_p(_ptr(weights)), _c_int(count), _c_void_p(_ptr(out)),
                   _c_ll(out.numel()))
        return out

    def stream_conv(self, residual, kernel, *, taps, ctx, view, sublayer, write, dtype):
        """What a sublayer reads of the 32-bit stream, in ``dtype``: x + its causal convolution
        over time on every channel (``kernel`` [hidden, taps]), the taps - 1 rows before a step's
        first token from row ``sublayer`` of the request's slot (``view``), where the step's last
        rows are left; without a kernel the stream, rounded."""
        self._need(residual, torch.float32, "residual")
        tokens, hidden = residual.shape
        out = torch.empty((tokens, hidden), dtype=dtype, device=self.device)
        state = slots = None
        stride = 0
        if kernel is None or taps < 1:
            kernel, taps = None, 0
        else:
            self._need(kernel, torch.float32, "kernel")
            if kernel.shape != (hidden, taps):
                raise KernelError("the convolution's weights are [hidden, taps]")
            if taps > 1:
                self._need(view.state, torch.float32, "state")
                if view.state.shape[2:] != (taps - 1, hidden):
                    raise KernelError("a slot keeps taps - 1 rows per sublayer")
                state, slots, stride = view.state[0, sublayer], view.slots, view.state.stride(0)
        self._call("mlxone_stream_conv", _c_void_p(_ptr(residual)), _c_void_p(_ptr(kernel)),
                   _c_int(taps), _c_void_p(_ptr(ctx.token_request)),
                   _c_void_p(_ptr(ctx.request_start)), _c_void_p(_ptr(state)), _c_ll(stride),
                   _c_void_p(_ptr(slots)), _c_void_p(_ptr(out)), _c_int(tokens), _c_int(hidden),
                   _c_int(1 if write else 0), _c_int(_dtype_code(dtype)))
        return out

    # ---- attention over one latent row per token; two score maps per head

    def latent_prepare(self, projected, queries, *, heads, head_dim, rot_dim, latent, norm_weight,
                       eps, rotary, neighbours, ctx, view, write):
        """The rotated parts of the queries into ``queries[:, :, latent:]``; the token's row
        [normed latent | rotated shared key part] into its request's pages."""
        self._need_rows(projected, queries.dtype, "projected")
        self._need(queries, queries.dtype, "queries")
        self._need(norm_weight, torch.float32, "norm weight")
        self._need(view.kv, queries.dtype, "pages")
        row = latent + rot_dim
        if queries.shape[1:] != (heads, row) or view.kv.shape[0] != 1 or \
                view.kv.shape[2] != 1 or view.kv.shape[-1] != row:
            raise KernelError("queries and pages hold rows of latent + rot_dim values")
        inv_freq, rotary_dim = (None, 0) if rotary is None else rotary
        self._call("mlxone_latent_prepare", _c_void_p(_ptr(projected)),
                   _c_int(projected.stride(0)), _c_void_p(_ptr(queries)),
                   _c_void_p(_ptr(norm_weight)), _c_float(eps), _c_void_p(_ptr(inv_freq)),
                   _c_int(rotary_dim), _c_int(1 if neighbours else 0),
                   _c_void_p(_ptr(ctx.positions)), _c_void_p(_ptr(ctx.token_request)),
                   _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(view.block_table)),
                   _c_int(view.block_table.shape[1]), _c_int(view.page_size),
                   _c_int(projected.shape[0]), _c_int(heads), _c_int(head_dim), _c_int(rot_dim),
                   _c_int(latent), _c_int(1 if write else 0), _c_int(_dtype_code(queries.dtype)),
                   _c_void_p(_ptr(self.error_flag)))

    def linear_heads(self, a, w, out=None):
        """a [tokens, heads, K] with w [heads, N, K] -> [tokens, heads, N], one product per head.
        The rows of ``a`` and ``out`` may be slices of wider rows (values of a head together)."""
        tokens, heads, k = a.shape
        n = w.shape[1]
        if w.shape != (heads, n, k) or a.stride(2) != 1 or a.dtype != w.dtype:
            raise KernelError("head-by-head product: a [tokens, heads, K], w [heads, N, K]")
        self._need(w, a.dtype, "w")
        if out is None:
            out = torch.empty((tokens, heads, n), dtype=a.dtype, device=self.device)
        if out.shape != (tokens, heads, n) or out.stride(2) != 1 or out.dtype != a.dtype:
            raise KernelError("head-by-head product: out [tokens, heads, N]")
        if tokens == 0:
            return out
        if a.dtype == torch.float32:
            self._call("mlxone_gemm_f32_batched", _c_void_p(_ptr(a)), _c_int(a.stride(0)),
                       _c_ll(a.stride(1)), _c_void_p(_ptr(w)), _c_int(k), _c_ll(n * k),
                       _c_void_p(_ptr(out)), _c_int(out.stride(0)), _c_ll(out.stride(1)),
                       _c_int(tokens), _c_int(n), _c_int(k), _c_int(heads))
        else:
            torch.bmm(a.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))
        return out

    def latent_attention(self, queries, *, heads, latent, scale, ctx, view):
        """Causal softmax attention of queries [tokens, heads, row] over the one row per token in
        the request's single-plane pages, which is key and value at once. Returns [tokens, heads,
        row]; the first ``latent`` values of a row are the weights' average of the latents.

        The bfloat16 kernel is launched as a programmatic dependent of the kernel ahead of it in
        the stream; before it waits for that kernel it reads ``ctx.positions``, the block table
        and rows of positions before the step's first (rows that earlier steps wrote)."""
        tokens, _, row = queries.shape
        self._need(queries, view.kv.dtype, "queries")
        out = torch.empty((tokens, heads, row), dtype=queries.dtype, device=self.device)
        if queries.dtype == torch.bfloat16 and \
                self.lib.mlxone_latent_attention_mma_fits(_c_int(row), _c_int(latent)):
            # tensor cores: blocks of 16 or 32 (token, head) rows that share the keys they read;
            # steps of single tokens cut the keys into runs that fill the GPU, merged afterwards
            splits, scratch = 1, None
            if ctx.max_portion == 1:
                blocks = ctx.requests * (1 if heads <= 16 else -(-heads // 32))
                bound = min(ctx.max_context, view.block_table.shape[1] * view.page_size)
                # as many runs as blocks fit on the GPU at once, two tiles a run where there are two, and
                # no run left without tiles (the kernel gives a run ceil(tiles / splits) tiles)
                tiles = -(-bound // 64)
                most = max(1, min(self._sm_count // blocks, -(-tiles // 2), 32))
                splits = -(-tiles // -(-tiles // most))
                if splits > 1:
                    scratch = torch.empty(splits * tokens * heads * (latent + 2),
                                          dtype=torch.float32, device=self.device)
            self._call("mlxone_latent_attention_mma", _c_void_p(_ptr(queries)),
                       _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(view.block_table)),
                       _c_int(view.block_table.shape[1]), _c_int(view.page_size),
                       _c_void_p(_ptr(ctx.positions)), _c_void_p(_ptr(ctx.request_start)),
                       _c_void_p(_ptr(out)), _c_void_p(_ptr(scratch)), _c_int(tokens),
                       _c_int(ctx.requests), _c_int(ctx.max_portion), _c_int(heads), _c_int(row),
                       _c_int(latent), _c_float(scale), _c_int(splits),
                       _c_void_p(_ptr(self.error_flag)))
            return out
        self._call("mlxone_attention_generic_planes", _c_void_p(_ptr(queries)),
                   _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(view.block_table)),
                   _c_int(view.block_table.shape[1]), _c_int(view.page_size),
                   _c_int(view.kv.shape[1]), _c_void_p(_ptr(ctx.positions)),
                   _c_void_p(_ptr(ctx.token_request)), _c_void_p(_ptr(out)), _c_int(tokens),
                   _c_int(heads), _c_int(1), _c_int(row), _c_float(scale), _c_int(0),
                   _c_int(_dtype_code(queries.dtype)), _c_void_p(None), _c_int(1),
                   _c_void_p(_ptr(self.error_flag)))
        return out

    def sigmoid_gate(self, values, gate):
        """values * sigmoid(gate); the gate's rows may be a slice of wider rows."""
        self._need(values, values.dtype, "values")
        self._need_rows(gate, values.dtype, "gate")
        if gate.shape != values.shape:
            raise KernelError("gate and values differ in shape")
        out = torch.empty_like(values)
        self._call("mlxone_sigmoid_gate", _c_void_p(_ptr(values)), _c_void_p(_ptr(gate)),
                   _c_int(gate.stride(0)), _c_void_p(_ptr(out)), _c_int(values.shape[0]),
                   _c_int(values.shape[1]), _c_int(_dtype_code(values.dtype)))
        return out

    def differential_combine(self, maps, *, heads, row_dim, value_dim, mix, eps, factor):
        """maps [tokens, 2 * heads * row_dim] (map by map, the first value_dim values of a row
        count) -> [tokens, heads * value_dim]: o = a1 - mix a2, o / rms(o) * factor, in 32-bit."""
        self._need(maps, maps.dtype, "maps")
        tokens = maps.shape[0]
        if maps.shape[1] != 2 * heads * row_dim:
            raise KernelError("the maps' width does not match the head count")
        out = torch.empty((tokens, heads * value_dim), dtype=maps.dtype, device=self.device)
        self._call("mlxone_differential_combine", _c_void_p(_ptr(maps)), _c_void_p(_ptr(out)),
                   _c_int(tokens), _c_int(heads), _c_int(row_dim), _c_int(value_dim),
                   _c_float(mix), _c_float(eps), _c_float(factor),
                   _c_int(_dtype_code(maps.dtype)))
        return out

    # ---- the 32-bit stream

    def add_vectors(self, residual, delta, token_ids, table, vector, delta_scale=1.0):
        """In place: residual[t] += delta_scale * delta[t] (if given) + table[token_ids[t]] (if a
        table is given) + vector (if given; float32 [hidden])."""
        self._need(residual, torch.float32, "residual")
        tokens, hidden = residual.shape
        code = _F32
        for tensor, what in ((delta, "delta"), (table, "table")):
            if tensor is not None:
                self._need(tensor, tensor.dtype, what)
                code = _dtype_code(tensor.dtype)
        if delta is not None and table is not None and delta.dtype != table.dtype:
            raise KernelError("delta and table differ in dtype")
        if delta is not None and delta.shape != residual.shape:
            raise KernelError("delta and residual differ in shape")
        if table is not None and table.shape[1] != hidden:
            raise KernelError("table rows and residual rows differ in length")
        if vector is not None:
            self._need(vector, torch.float32, "vector")
            if vector.numel() != hidden:
                raise KernelError("vector and residual rows differ in length")
        self._call("mlxone_add_vectors", _c_void_p(_ptr(residual)), _c_void_p(_ptr(delta)),
                   _c_void_p(_ptr(token_ids)), _c_void_p(_ptr(table)), _c_void_p(_ptr(vector)),
                   _c_int(tokens), _c_int(hidden),
                   _c_int(0 if table is None else table.shape[0]), _c_int(code),
                   _c_float(delta_scale))

    def concat_stream(self, residual, delta, token_ids, table, dtype, delta_scale=1.0):
        """[tokens, 2 hidden] in ``dtype``: the stream (with delta_scale * delta, if given) beside
        the tokens' rows of ``table``."""
        self._need(residual, torch.float32, "residual")
        self._need(table, dtype, "table")
        self._need(token_ids, torch.int32, "token ids")
        tokens, hidden = residual.shape
        if delta is not None:
            self._need(delta, dtype, "delta")
            if delta.shape != residual.shape:
                raise KernelError("delta and residual differ in shape")
        if table.shape[1] != hidden:
            raise KernelError("table rows and residual rows differ in length")
        out = torch.empty((tokens, 2 * hidden), dtype=dtype, device=self.device)
        self._call("mlxone_concat_stream", _c_void_p(_ptr(residual)), _c_void_p(_ptr(delta)),
                   _c_void_p(_ptr(token_ids)), _c_void_p(_ptr(table)), _c_void_p(_ptr(out)),
                   _c_int(tokens), _c_int(hidden), _c_int(table.shape[0]),
                   _c_int(_dtype_code(dtype)), _c_float(delta_scale))
        return out

    def softcap(self, logits, cap):
        """In place: logits = cap * tanh(logits / cap) (float32)."""
        self._need(logits, torch.float32, "logits")
        self._call("mlxone_softcap", _c_void_p(_ptr(logits)), _c_ll(logits.numel()), _c_float(cap))

    # ---- routed experts

    def route_experts(self, x, router, *, experts, top, groups, keep, group_score):
        """Routing weights float32 [tokens, experts] (zero for experts that were not chosen):
        sigmoid scores of the 32-bit logits, the ``keep`` best of ``groups`` groups by the sum of
        their ``group_score`` largest scores, the ``top`` best of their experts, normalised."""
        self._need_rows(x, x.dtype, "x")
        self._need(router, torch.float32, "router")
        if router.shape != (experts, x.shape[1]):
            raise KernelError("the router's shape does not match")
        weights = torch.empty((x.shape[0], experts), dtype=torch.float32, device=self.device)
        self._call("mlxone_route_experts", _c_void_p(_ptr(x)), _c_int(x.stride(0)),
                   _c_void_p(_ptr(router)), _c_void_p(_ptr(weights)), _c_int(x.shape[0]),
                   _c_int(x.shape[1]), _c_int(experts), _c_int(top), _c_int(groups), _c_int(keep),
                   _c_int(group_score), _c_int(_dtype_code(x.dtype)))
        return weights

    def scale_expert_columns(self, gated, weights, width, tail=None):
        """In place: gated[t, e * width + f] *= weights[t, e]; columns beyond the experts' stay,
        or, with ``tail`` (float32 [tokens]), are multiplied by tail[t] (a shared expert's gate)."""
        self._need_rows(gated, gated.dtype, "gated")
        self._need(weights, torch.float32, "weights")
        if tail is not None:
            self._need(tail, torch.float32, "tail")
            rest = gated.shape[1] - weights.shape[1] * width
            if tail.numel() != gated.shape[0] or rest < 0:
                raise KernelError("one factor per token for the columns behind the experts'")
            self._call("mlxone_scale_expert_columns_tail", _c_void_p(_ptr(gated)),
                       _c_int(gated.stride(0)), _c_void_p(_ptr(weights)), _c_int(gated.shape[0]),
                       _c_int(weights.shape[1]), _c_int(width), _c_void_p(_ptr(tail)), _c_int(rest),
                       _c_int(_dtype_code(gated.dtype)))
            return
        self._call("mlxone_scale_expert_columns", _c_void_p(_ptr(gated)), _c_int(gated.stride(0)),
                   _c_void_p(_ptr(weights)), _c_int(gated.shape[0]), _c_int(weights.shape[1]),
                   _c_int(width), _c_int(_dtype_code(gated.dtype)))

    def route_general(self, x, router, correction, *, experts, identity, top, scores, normalize,
                      shared_gate):
        """The second routing kernel. ``router`` float32 [experts + identity (+ 1 with
        ``shared_gate``), hidden]; scores are the sigmoid of the 32-bit logits or their softmax
        over the experts + identity outputs; ``correction`` (float32 per output, or None) is
        added where the ``top`` best are chosen; the weights are the chosen scores, divided by
        their sum with ``normalize``. Returns (weights float32 [tokens, experts], zero where an
        expert was not chosen; others float32 [2, tokens]: the sum of the chosen identity
        outputs' weights, and the sigmoid of the router's last row's logit, 1 without
        ``shared_gate``)."""
        self._need_rows(x, x.dtype, "x")
        self._need(router, torch.float32, "router")
        rows = experts + identity + (1 if shared_gate else 0)
        if router.shape != (rows, x.shape[1]):
            raise KernelError("the router's shape does not match")
        if scores not in ("sigmoid", "softmax"):
            raise KernelError(f"unknown routing scores {scores!r}")
        if correction is not None:
            self._need(correction, torch.float32, "correction")
            if correction.numel() != experts + identity:
                raise KernelError("one correction per output of the router")
        tokens = x.shape[0]
        weights = torch.empty((tokens, experts), dtype=torch.float32, device=self.device)
        others = torch.empty((2, tokens), dtype=torch.float32, device=self.device)
        self._call("mlxone_route_general", _c_void_p(_ptr(x)), _c_int(x.stride(0)),
                   _c_void_p(_ptr(router)), _c_void_p(_ptr(correction)), _c_void_p(_ptr(weights)),
                   _c_void_p(_ptr(others)), _c_int(tokens), _c_int(x.shape[1]), _c_int(experts),
                   _c_int(identity), _c_int(top), _c_int(1 if scores == "softmax" else 0),
                   _c_int(1 if normalize else 0), _c_int(1 if shared_gate else 0),
                   _c_int(_dtype_code(x.dtype)))
        return weights, others

    def add_scaled_rows(self, out, x, factors):
        """In place: out[t] += factors[t] * x[t] (32-bit sum, stored in out's dtype)."""
        self._need(out, out.dtype, "out")
        self._need_rows(x, out.dtype, "x")
        self._need(factors, torch.float32, "factors")
        if x.shape != out.shape or factors.numel() != out.shape[0]:
            raise KernelError("rows, their source and one factor per row must match")
        self._call("mlxone_add_scaled_rows", _c_void_p(_ptr(out)), _c_void_p(_ptr(x)),
                   _c_int(x.stride(0)), _c_void_p(_ptr(factors)), _c_int(out.shape[0]),
                   _c_int(out.shape[1]), _c_int(_dtype_code(out.dtype)))

    def scale_values(self, values, factor):
        """In place: values *= factor (float32)."""
        self._need(values, torch.float32, "values")
        self._call("mlxone_scale_values", _c_void_p(_ptr(values)), _c_ll(values.numel()),
                   _c_float(factor))

    # ---- convolutions over time on the channels of a projection; the selective state space

    def channel_conv(self, rows, kernel, bias, *, taps, activation, ctx, view, write):
        """act(sum_j kernel[:, j] * rows_(t - taps + 1 + j) + bias) over each request's tokens;
        the taps - 1 rows before a step's first token come from the request's slot (``view``:
        [slots, taps - 1, channels] in the rows' dtype), where the step's last rows are left.
        ``rows`` may be a slice of wider rows; the result has rows of its own. ``activation``:
        None or ``silu``. A step of single tokens is one kernel, else the convolution and the
        slots' update."""
        self._need_rows(rows, rows.dtype, "rows")
        tokens, channels = rows.shape
        self._need(kernel, torch.float32, "conv kernel")
        if kernel.shape != (channels, taps):
            raise KernelError("the convolution's weights are [channels, taps]")
        if bias is not None:
            self._need(bias, torch.float32, "conv bias")
        if activation not in (None, "silu"):
            raise KernelError(f"unknown activation {activation!r}")
        state = slots = None
        if taps > 1:
            self._need(view.state, rows.dtype, "state")
            if view.state.shape[1:] != (taps - 1, channels):
                raise KernelError("a slot keeps taps - 1 rows of the convolution's inputs")
            state, slots = view.state, view.slots
        out = torch.empty((tokens, channels), dtype=rows.dtype, device=self.device)
        single = ctx.max_portion == 1 and tokens == ctx.requests
        self._call("mlxone_channel_conv", _c_void_p(_ptr(rows)), _c_int(rows.stride(0)),
                   _c_void_p(_ptr(kernel)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(state)),
                   _c_void_p(_ptr(slots)), _c_void_p(_ptr(ctx.token_request)),
                   _c_void_p(_ptr(ctx.request_start)), _c_void_p(_ptr(ctx.history)),
                   _c_void_p(_ptr(out)), _c_int(tokens), _c_int(ctx.requests), _c_int(channels),
                   _c_int(taps), _c_int(1 if activation == "silu" else 0),
                   _c_int(1 if single else 0), _c_int(1 if write else 0),
                   _c_int(_dtype_code(rows.dtype)))
        if not single and write and taps > 1:
            self.launches += 1
        return out

    def state_space_scan(self, mixed, steps, *, a_log, dt_bias, skip, ctx, view, write, heads,
                         value_dim, state_dim, groups):
        """The recurrence of a selective state space. ``mixed`` [tokens, x | B | C] (heads *
        value_dim, then twice groups * state_dim) and ``steps`` [tokens, heads] (raw step sizes,
        may be a slice of wider rows) in the compute dtype; dt = softplus(steps + dt_bias),
        S = exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + skip x over each request's tokens on
        its 32-bit state [heads, state_dim, value_dim]. Returns y float32 [tokens, heads *
        value_dim]."""
        tokens = mixed.shape[0]
        self._need(mixed, mixed.dtype, "mixed")
        self._need_rows(steps, mixed.dtype, "steps")
        inner = heads * value_dim
        if mixed.shape[1] != inner + 2 * groups * state_dim or steps.shape != (tokens, heads):
            raise KernelError("the convolution's width does not match the head counts")
        for tensor, what in ((a_log, "A_log"), (dt_bias, "dt_bias"), (skip, "D"),
                             (view.state, "state")):
            self._need(tensor, torch.float32, what)
        if view.state[0].numel() != heads * state_dim * value_dim:
            raise KernelError(f"a state slot has {view.state[0].numel()} values, the mixer needs "
                              f"{heads * state_dim * value_dim}")
        scratch = torch.empty(self.lib.mlxone_state_space_scratch(
            tokens, ctx.requests, ctx.max_portion, heads, value_dim, state_dim),
            dtype=torch.float32, device=self.device)
        y = torch.empty((tokens, inner), dtype=torch.float32, device=self.device)
        self._call("mlxone_state_space_scan", _c_void_p(_ptr(mixed)), _c_void_p(_ptr(steps)),
                   _c_int(steps.stride(0)), _c_void_p(_ptr(a_log)), _c_void_p(_ptr(dt_bias)),
                   _c_void_p(_ptr(skip)), _c_void_p(_ptr(view.state)), _c_void_p(_ptr(view.slots)),
                   _c_void_p(_ptr(ctx.request_start)), _c_void_p(_ptr(scratch)),
                   _c_void_p(_ptr(y)), _c_int(tokens), _c_int(ctx.requests),
                   _c_int(ctx.max_portion), _c_int(heads), _c_int(value_dim), _c_int(state_dim),
                   _c_int(groups), _c_int(1 if write else 0), _c_int(_dtype_code(mixed.dtype)))
        if ctx.max_portion >= 128:
            self.launches += 2
        return y

    def gated_group_norm(self, y, gate, weight, *, groups, eps, dtype):
        """(y * silu(gate)) divided by its root mean square in ``groups`` equal parts of a row
        (each part by its own), times ``weight``; y float32 [tokens, inner], the gate's rows in
        ``dtype`` (may be a slice of wider rows); the result in ``dtype``."""
        self._need(y, torch.float32, "y")
        self._need_rows(gate, dtype, "gate")
        self._need(weight, torch.float32, "norm weight")
        tokens, inner = y.shape
        if gate.shape != y.shape or weight.numel() != inner or inner % groups:
            raise KernelError("gate, weight and the norm's parts must match the rows")
        out = torch.empty((tokens, inner), dtype=dtype, device=self.device)
        self._call("mlxone_gated_group_norm", _c_void_p(_ptr(y)), _c_void_p(_ptr(gate)),
                   _c_int(gate.stride(0)), _c_void_p(_ptr(weight)), _c_void_p(_ptr(out)),
                   _c_int(tokens), _c_int(inner), _c_int(groups), _c_float(eps),
                   _c_int(_dtype_code(dtype)))
        return out

    def gate_heads(self, mixed, gate, *, heads, row_dim, value_dim, per_head):
        """The heads' outputs [tokens, heads * row_dim] (the first ``value_dim`` values of a
        head's row count) times sigmoid(gate), one number per value or, with ``per_head``, per
        head -> [tokens, heads * value_dim]. The gate's rows may be a slice of wider rows."""
        self._need(mixed, mixed.dtype, "mixed")
        self._need_rows(gate, mixed.dtype, "gate")
        tokens = mixed.shape[0]
        if mixed.shape[1] != heads * row_dim or \
                gate.shape != (tokens, heads * (1 if per_head else value_dim)):
            raise KernelError("the gate does not match the heads' outputs")
        out = torch.empty((tokens, heads * value_dim), dtype=mixed.dtype, device=self.device)
        self._call("mlxone_gate_heads", _c_void_p(_ptr(mixed)), _c_void_p(_ptr(gate)),
                   _c_int(gate.stride(0)), _c_void_p(_ptr(out)), _c_int(tokens), _c_int(heads),
                   _c_int(row_dim), _c_int(value_dim), _c_int(1 if per_head else 0),
                   _c_int(_dtype_code(mixed.dtype)))
        return out

    # Steps of at least this many tokens run routed experts over tokens sorted by expert (grouped
    # tcgen05 products that touch only the experts a token uses), and so do steps so small that
    # their tokens use at most half of the experts (a single token that uses 2 of 8, or 6 of 64,
    # should not read them all); the steps between run every token through all experts in one
    # stacked product, which reads the same weights at those sizes with fewer launches.
    sorted_experts_min_tokens = 128

    def sorts_experts(self, x, *, experts, width, top, stack) -> bool:
        """Whether ``routed_experts_sorted`` takes this step."""
        tokens = x.shape[0]
        return (self.tcgen05_products and x.dtype == torch.bfloat16 and top < experts
                and (tokens >= self.sorted_experts_min_tokens or 2 * tokens * top <= experts)
                and x.shape[1] % 8 == 0 and width % 8 == 0 and stack % 8 == 0
                and x.stride(1) == 1 and x.stride(0) % 8 == 0)

    def routed_experts_sorted(self, x, weights, gate_up, down, *, experts, width, top,
                              shared_gate_up=None, shared_down=None, shared_scale=None):
        """The weighted sum of every token's chosen experts (+ the shared expert's output), with
        the tokens sorted by expert: gate_up [2 stack, hidden] holds the experts' gate rows, then
        (``stack`` rows further) their up rows; down [hidden, stack] their down matrices side by
        side. weights [tokens, experts] float32, zero where an expert was not chosen."""
        tokens, hidden = x.shape
        stack = gate_up.shape[0] // 2
        tiles = -(-(tokens * top + experts * 127) // 128)
        rows = tiles * 128
        pair_row = torch.empty((tokens, experts), dtype=torch.int32, device=self.device)
        groups = torch.empty((2, tiles, 2), dtype=torch.int32, device=self.device)
        self._call("mlxone_sort_by_expert", _c_void_p(_ptr(weights)), _c_void_p(_ptr(pair_row)),
                   _c_void_p(_ptr(groups)), _c_int(tokens), _c_int(experts), _c_int(width),
                   _c_int(tiles))
        # (rows that no pair owns are multiplied like the others, but nothing reads their results,
        # and a row's result depends on no other row: they need no values of their own)
        sorted_x = torch.empty((rows, hidden), dtype=x.dtype, device=self.device)
        self._call("mlxone_gather_by_expert", _c_void_p(_ptr(x)), _c_int(x.stride(0)),
                   _c_void_p(_ptr(pair_row)), _c_void_p(_ptr(sorted_x)), _c_int(tokens),
                   _c_int(hidden), _c_int(experts), _c_int(_dtype_code(x.dtype)))
        gated = torch.empty((rows, width), dtype=x.dtype, device=self.device)
        self._call("mlxone_gemm_tcgen05_grouped", _c_void_p(_ptr(sorted_x)), _c_int(hidden),
                   _c_void_p(_ptr(gate_up)), _c_ll(gate_up.shape[0]), _c_ll(hidden), _c_ll(hidden),
                   _c_void_p(_ptr(gated)), _c_int(width), _c_int(rows), _c_int(width),
                   _c_int(hidden), _c_int(stack), _c_int(self._SWIGLU),
                   _c_void_p(_ptr(groups[0])), _c_void_p(_ptr(self.error_flag)))
        y = torch.empty((rows, hidden), dtype=x.dtype, device=self.device)
        self._call("mlxone_gemm_tcgen05_grouped", _c_void_p(_ptr(gated)), _c_int(width),
                   _c_void_p(_ptr(down)), _c_ll(hidden), _c_ll(stack), _c_ll(stack),
                   _c_void_p(_ptr(y)), _c_int(hidden), _c_int(rows), _c_int(hidden), _c_int(width),
                   _c_int(0), _c_int(self._STORE), _c_void_p(_ptr(groups[1])),
                   _c_void_p(_ptr(self.error_flag)))
        shared_out = None
        if shared_gate_up is not None:
            shared_gated = self.linear_swiglu(x, shared_gate_up)
            if shared_scale is not None:
                # (one number per token on the shared expert's output, applied ahead of its down
                # product, which is linear)
                self.scale_expert_columns(shared_gated, shared_scale.view(-1, 1),
                                          shared_gated.shape[1])
            shared_out = self.linear(shared_gated, shared_down)
        out = torch.empty((tokens, hidden), dtype=x.dtype, device=self.device)
        self._call("mlxone_combine_experts", _c_void_p(_ptr(y)), _c_void_p(_ptr(pair_row)),
                   _c_void_p(_ptr(weights)), _c_void_p(_ptr(shared_out)), _c_void_p(_ptr(out)),
                   _c_int(tokens), _c_int(hidden), _c_int(experts), _c_int(_dtype_code(x.dtype)))
        return out

    # ---- lightning attention

    def lightning_attention(self, projected, *, decay, norm_weight, eps, ctx, view, write, heads,
                            key_dim, value_dim):
        """From the fused projection [tokens, q | k | v | gate] to the mixer's gated output
        [tokens, heads * value_dim]: silu, the recurrence S = decay S + k v^T, o = S^T q over each
        request's tokens on its 32-bit state [heads, key_dim, value_dim], the norm over all heads
        and the sigmoid gate."""
        tokens = projected.shape[0]
        self._need_rows(projected, projected.dtype, "projected")
        inner = heads * value_dim
        if projected.shape[1] != 2 * heads * key_dim + 2 * inner:
            raise KernelError("the projection's width does not match the head counts")
        for tensor, what in ((decay, "decay"), (norm_weight, "norm weight"), (view.state, "state")):
            self._need(tensor, torch.float32, what)
        if view.state[0].numel() != heads * key_dim * value_dim:
            raise KernelError(f"a state slot has {view.state[0].numel()} values, the mixer needs "
                              f"{heads * key_dim * value_dim}")
        scratch = torch.empty(self.lib.mlxone_lightning_scratch(
            tokens, ctx.requests, ctx.max_portion, heads, key_dim, value_dim),
            dtype=torch.float32, device=self.device)
        out = torch.empty((tokens, inner), dtype=projected.dtype, device=self.device)
        self._call("mlxone_lightning", _c_void_p(_ptr(projected)), _c_int(projected.stride(0)),
                   _c_void_p(_ptr(decay)), _c_void_p(_ptr(norm_weight)), _c_float(eps),
                   _c_void_p(_ptr(view.state)), _c_void_p(_ptr(view.slots)),
                   _c_void_p(_ptr(ctx.request_start)), _c_void_p(_ptr(scratch)),
                   _c_void_p(_ptr(out)), _c_int(tokens), _c_int(ctx.requests),
                   _c_int(ctx.max_portion), _c_int(heads), _c_int(key_dim), _c_int(value_dim),
                   _c_int(1 if write else 0), _c_int(_dtype_code(projected.dtype)))
        self.launches += 1 if ctx.max_portion < 128 else 3
        return out

    def normed_mean_add(self, residual, outputs, weights, eps):
        """In place: residual += mean over branches of x / rms(x) * weight (rms over the row,
        eps inside the root), all in 32-bit."""
        self._need(residual, torch.float32, "residual")
        count = len(outputs)
        if not 1 <= count <= 4 or len(weights) != count:
            raise KernelError("one to four branches, each with a weight")
        for x, weight in zip(outputs, weights):
            self._need(x, outputs[0].dtype, "branch output")
            self._need(weight, torch.float32, "branch weight")
            if x.shape != residual.shape or weight.numel() != residual.shape[1]:
                raise KernelError("branch outputs and weights must match the residual")
        xs = (ctypes.c_void_p * count)(*[x.data_ptr() for x in outputs])
        ws = (ctypes.c_void_p * count)(*[w.data_ptr() for w in weights])
        self._call("mlxone_normed_mean_add", _c_void_p(_ptr(residual)), xs, ws, _c_int(count),
                   _c_int(residual.shape[0]), _c_int(residual.shape[1]), _c_float(eps),
                   _c_int(_dtype_code(outputs[0].dtype)))

    # ---- the gated delta rule

    def gated_delta_rule(self, projected, *, conv, a_log, dt_bias, norm_weight, eps, unit_eps, ctx,
                         view, write, heads, kv_heads, key_dim, value_dim, taps):
        """From the fused projection [tokens, q | k | v | gate | beta | decay] to the mixer's
        gated output [tokens, heads * value_dim]: convolutions with silu, unit-length queries
        and keys, the recurrence over each request's tokens on its 32-bit state, the output's
        norm and gate. The state slot holds the heads' matrices and a ring of the convolutions'
        inputs (row position % taps)."""
        tokens = projected.shape[0]
        self._need_rows(projected, projected.dtype, "projected")
        qk, inner = kv_heads * key_dim, heads * value_dim
        if projected.shape[1] != 2 * qk + 2 * inner + 2 * heads:
            raise KernelError("the projection's width does not match the head counts")
        for tensor, what in ((conv, "conv"), (a_log, "A_log"), (dt_bias, "dt_bias"),
                             (norm_weight, "norm weight"), (view.state, "state")):
            self._need(tensor, torch.float32, what)
        size = self.lib.mlxone_gated_delta_state(heads, kv_heads, key_dim, value_dim, taps)
        if view.state[0].numel() != size:
            raise KernelError(f"a state slot has {view.state[0].numel()} values, the mixer needs {size}")
        # a step of single tokens runs as one kernel, else preparation, scan and finish
        single = ctx.max_portion == 1 and tokens == ctx.requests
        scratch = torch.empty(self.lib.mlxone_gated_delta_scratch(tokens, heads, kv_heads, key_dim,
                                                                  value_dim),
                              dtype=torch.float32, device=self.device)
        out = torch.empty((tokens, inner), dtype=projected.dtype, device=self.device)
        self._call("mlxone_gated_delta", _c_void_p(_ptr(projected)), _c_void_p(_ptr(conv)),
                   _c_void_p(_ptr(a_log)), _c_void_p(_ptr(dt_bias)), _c_void_p(_ptr(norm_weight)),
                   _c_float(eps), _c_float(unit_eps), _c_void_p(_ptr(view.state)),
                   _c_void_p(_ptr(view.slots)), _c_void_p(_ptr(ctx.token_request)),
                   _c_void_p(_ptr(ctx.request_start)), _c_void_p(_ptr(ctx.history)),
                   _c_void_p(_ptr(scratch)), _c_void_p(_ptr(out)), _c_int(tokens),
                   _c_int(ctx.requests), _c_int(heads), _c_int(kv_heads), _c_int(key_dim),
                   _c_int(value_dim), _c_int(taps), _c_int(1 if write else 0),
                   _c_int(projected.stride(0)), _c_int(1 if single else 0),
                   _c_int(_dtype_code(projected.dtype)))
        if not (single and value_dim <= 128):
            self.launches += 2
        return out

    def swiglu(self, gate_up):
        rows, twice = gate_up.shape
        out = torch.empty((rows, twice // 2), dtype=gate_up.dtype, device=self.device)
        self._call("mlxone_swiglu", _c_void_p(_ptr(gate_up)), _c_void_p(_ptr(out)), _c_int(rows),
                   _c_int(twice // 2), _c_int(_dtype_code(gate_up.dtype)))
        return out

    def short_conv(self, bcx, *, kernel, bias, taps, ctx, view, write):
        tokens, triple = bcx.shape
        hidden = triple // 3
        self._need(bcx, view.state.dtype, "bcx")
        self._need(kernel, torch.float32, "conv kernel")
        out = torch.empty((tokens, hidden), dtype=bcx.dtype, device=self.device)
        if ctx.max_portion == 1 and tokens == ctx.requests:
            # decode: output and state update in one kernel
            self._call("mlxone_short_conv_decode", _c_void_p(_ptr(bcx)), _c_void_p(_ptr(kernel)),
                       _c_void_p(_ptr(bias)), _c_void_p(_ptr(view.state)),
                       _c_void_p(_ptr(view.slots)), _c_void_p(_ptr(ctx.history)),
                       _c_void_p(_ptr(out)), _c_int(tokens), _c_int(hidden), _c_int(taps),
                       _c_int(1 if write else 0), _c_int(_dtype_code(bcx.dtype)))
            return out
        self._call("mlxone_short_conv", _c_void_p(_ptr(bcx)), _c_void_p(_ptr(kernel)),
                   _c_void_p(_ptr(bias)), _c_void_p(_ptr(view.state)), _c_void_p(_ptr(view.slots)),
                   _c_void_p(_ptr(ctx.token_request)), _c_void_p(_ptr(ctx.request_start)),
                   _c_void_p(_ptr(ctx.history)), _c_void_p(_ptr(out)), _c_int(tokens),
                   _c_int(ctx.requests), _c_int(hidden), _c_int(taps), _c_int(1 if write else 0),
                   _c_int(_dtype_code(bcx.dtype)))
        return out

    def linear_short_conv(self, a, w, w_bias, *, kernel, bias, taps, ctx, view, write):
        """short_conv(linear(a, w, w_bias)): for a decode step of few rows one kernel, the
        convolution's update being the product's epilogue; else the two operations."""
        fits = (ctx.max_portion == 1 and a.shape[0] == ctx.requests and taps <= 4
                and w.shape[0] % 3 == 0 and view.state.dtype == torch.bfloat16)
        if (isinstance(a, NormedInput) and fits and self.lib.mlxone_gemm_skinny_conv_norm_fits(
                _c_int(a.shape[0]), _c_int(a.shape[1]))):
            # the norm while the rows are loaded, the product, the convolution's update: one kernel
            self._need(w, torch.bfloat16, "w")
            self._need(kernel, torch.float32, "conv kernel")
            if w.shape[1] != a.residual.shape[1]:
                raise KernelError(f"matrix product of {tuple(a.shape)} with {tuple(w.shape)}^T")
            hidden = w.shape[0] // 3
            out = torch.empty((a.shape[0], hidden), dtype=a.dtype, device=self.device)
            self._call("mlxone_gemm_skinny_conv_norm", _c_void_p(_ptr(a.residual)),
                       _c_int(a.residual.stride(0)), _c_void_p(_ptr(a.weight)), _c_float(a.eps),
                       _c_void_p(_ptr(w)), _c_void_p(_ptr(w_bias)), _c_void_p(_ptr(out)),
                       _c_int(a.shape[0]), _c_int(hidden), _c_int(a.shape[1]),
                       _c_void_p(_ptr(kernel)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(view.state)),
                       _c_void_p(_ptr(view.slots)), _c_void_p(_ptr(ctx.history)), _c_int(taps),
                       _c_int(1 if write else 0))
            return out
        if not isinstance(a, NormedInput) and fits and self._skinny(a, w, fused=True):
            self._check_product(a, w)
            self._need(kernel, torch.float32, "conv kernel")
            hidden = w.shape[0] // 3
            out = torch.empty((a.shape[0], hidden), dtype=a.dtype, device=self.device)
            self._call("mlxone_gemm_skinny_conv", _c_void_p(_ptr(a)), _c_int(a.stride(0)),
                       _c_void_p(_ptr(w)), _c_void_p(_ptr(w_bias)), _c_void_p(_ptr(out)),
                       _c_int(a.shape[0]), _c_int(hidden), _c_int(a.shape[1]),
                       _c_void_p(_ptr(kernel)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(view.state)),
                       _c_void_p(_ptr(view.slots)), _c_void_p(_ptr(ctx.history)), _c_int(taps),
                       _c_int(1 if write else 0))
            return out
        return self.short_conv(self.linear(a, w, w_bias), kernel=kernel, bias=bias, taps=taps,
                               ctx=ctx, view=view, write=write)

    def qk_norm_rope_store(self, qkv, *, heads, kv_heads, head_dim, q_weight, k_weight, eps,
                           rotary, ctx, view, write, value_dim=None, amplitude=1.0,
                           norm_after=False):
        """Queries [tokens, heads, row] ready for attention; keys and values written to the
        pages. ``value_dim``, ``amplitude`` (a factor on cosine and sine) and ``norm_after``
        (queries and keys divided by their root mean square after the rotation, no weight)
        select the general kernel, which pads queries, keys and values with zeros to the
        pages' row size."""
        tokens = qkv.shape[0]
        inv_freq, rotary_dim = (None, 0) if rotary is None else rotary
        row_dim = view.kv.shape[-1]
        value_dim = value_dim or head_dim
        general = value_dim != head_dim or row_dim != head_dim or amplitude != 1.0 or norm_after
        if general:
            self._need_rows(qkv, view.kv.dtype, "qkv")
        else:
            self._need(qkv, view.kv.dtype, "qkv")
        if general:
            if qkv.shape[1] != (heads + kv_heads) * head_dim + kv_heads * value_dim:
                raise KernelError("qkv width does not match the head counts")
            if norm_after and eps is None:
                raise KernelError("a norm after the rotation needs its eps")
            mode = 2 if norm_after else (1 if q_weight is not None else 0)
            q = torch.empty((tokens, heads, row_dim), dtype=qkv.dtype, device=self.device)
            self._call("mlxone_qk_prep_general", _c_void_p(_ptr(qkv)), _c_void_p(_ptr(q_weight)),
                       _c_void_p(_ptr(k_weight)), _c_float(0.0 if eps is None else eps),
                       _c_void_p(_ptr(inv_freq)), _c_int(rotary_dim), _c_float(amplitude),
                       _c_int(mode), _c_void_p(_ptr(ctx.positions)),
                       _c_void_p(_ptr(ctx.token_request)), _c_void_p(_ptr(q)),
                       _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(view.block_table)),
                       _c_int(view.block_table.shape[1]), _c_int(view.page_size),
                       _c_int(view.kv.shape[1]), _c_int(tokens), _c_int(heads), _c_int(kv_heads),
                       _c_int(head_dim), _c_int(value_dim), _c_int(row_dim),
                       _c_int(1 if write else 0), _c_int(qkv.stride(0)),
                       _c_int(_dtype_code(qkv.dtype)),
                       _c_void_p(_ptr(self.error_flag)))
            return q
        if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
            raise KernelError("qkv width does not match the head counts")
        q = torch.empty((tokens, heads, head_dim), dtype=qkv.dtype, device=self.device)
        pages = view.kv.shape[1]
        self._call("mlxone_qk_prep", _c_void_p(_ptr(qkv)), _c_void_p(_ptr(q_weight)),
                   _c_void_p(_ptr(k_weight)), _c_float(0.0 if eps is None else eps),
                   _c_void_p(_ptr(inv_freq)), _c_int(rotary_dim), _c_void_p(_ptr(ctx.positions)),
                   _c_void_p(_ptr(ctx.token_request)), _c_void_p(_ptr(q)),
                   _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(view.block_table)),
                   _c_int(view.block_table.shape[1]), _c_int(view.page_size), _c_int(pages),
                   _c_int(tokens), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
                   _c_int(1 if write else 0), _c_int(_dtype_code(qkv.dtype)),
                   _c_void_p(_ptr(self.error_flag)))
        return q

    @staticmethod
    def _span(window, chunk):
        """What the attention kernels take as their window: a positive number of keys for a
        sliding window, minus the chunk size for chunks of positions that see only themselves,
        0 for every earlier key."""
        if window and chunk:
            raise KernelError("a window and chunks together are not implemented")
        return -int(chunk) if chunk else int(window or 0)

    def qkv_attention(self, qkv, *, heads, kv_heads, head_dim, q_weight, k_weight, eps, rotary,
                      scale, window, ctx, view, write, sinks=None, chunk=None, keep_first=0,
                      **extra):
        """From the fused projection qkv [tokens, (heads + 2 kv_heads) * head_dim] to the mixed
        heads [tokens, heads * head_dim]: per-head norm of queries and keys, rotation, keys and
        values appended to the pages, attention. A step of single tokens in bfloat16 whose head
        size is a multiple of 32 and whose rotation covers the whole head (or is none) runs as
        one kernel; everything else as the preparation kernel followed by attention."""
        tokens = qkv.shape[0]
        inv_freq, rotary_dim = (None, 0) if rotary is None else rotary
        window = self._span(window, chunk)
        if extra:
            # (value size, amplitude, norm after the rotation: see qk_norm_rope_store) the
            # general preparation, then attention over rows of the pages' size; the output has
            # that row size per head, zeros behind the values
            q = self.qk_norm_rope_store(qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                        q_weight=q_weight, k_weight=k_weight, eps=eps,
                                        rotary=rotary, ctx=ctx, view=view, write=write, **extra)
            return self.paged_attention(q, heads=heads, kv_heads=kv_heads,
                                        head_dim=view.kv.shape[-1], scale=scale, window=window,
                                        ctx=ctx, view=view, sinks=sinks, keep_first=keep_first)
        if (self.fused_decode_attention and qkv.dtype == torch.bfloat16
                and ctx.max_portion == 1 and tokens == ctx.requests
                and self.tensor_core_attention and not keep_first
                and self.lib.mlxone_attention_decode_fused_supports(_c_int(head_dim))
                and (inv_freq is None or rotary_dim == head_dim)
                and (q_weight is None) == (k_weight is None)):
            self._need(qkv, view.kv.dtype, "qkv")
            if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
                raise KernelError("qkv width does not match the head counts")
            out = torch.empty((tokens, heads * head_dim), dtype=qkv.dtype, device=self.device)
            width = view.block_table.shape[1]
            splits, partial = self._decode_plan(tokens, heads, kv_heads, head_dim, width, window,
                                                view)
            self._call("mlxone_attention_decode_fused", _c_void_p(_ptr(qkv)),
                       _c_void_p(_ptr(q_weight)), _c_void_p(_ptr(k_weight)),
                       _c_float(0.0 if eps is None else eps), _c_void_p(_ptr(inv_freq)),
                       _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(view.block_table)), _c_int(width),
                       _c_int(view.page_size), _c_int(view.kv.shape[1]),
                       _c_void_p(_ptr(ctx.positions)), _c_void_p(_ptr(out)),
                       _c_void_p(_ptr(partial)), _c_int(tokens), _c_int(heads), _c_int(kv_heads),
                       _c_int(head_dim), _c_int(splits), _c_float(scale), _c_int(window),
                       _c_int(1 if write else 0), _c_void_p(_ptr(sinks)),
                       _c_void_p(_ptr(self.error_flag)))
            if partial is not None:
                self.launches += 1          # the merge kernel
            return out
        q = self.qk_norm_rope_store(qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                    q_weight=q_weight, k_weight=k_weight, eps=eps, rotary=rotary,
                                    ctx=ctx, view=view, write=write)
        return self.paged_attention(q, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                    scale=scale, window=window, ctx=ctx, view=view, sinks=sinks,
                                    keep_first=keep_first)

    def paged_attention(self, q, *, heads, kv_heads, head_dim, scale, window, ctx, view,
                        sinks=None, chunk=None, keep_first=0):
        """Attention of every token over its request's pages. ``keep_first``: behind a window the
        first ``keep_first`` positions of a sequence stay visible. bfloat16 with a head size that
        is a multiple of 16 up to 128 runs on tensor cores: the split-key decode kernel when
        every request brings one token, else the prefill kernel. Everything else (float32,
        other head sizes) runs the general kernel."""
        tokens = q.shape[0]
        out = torch.empty((tokens, heads * head_dim), dtype=q.dtype, device=self.device)
        width = view.block_table.shape[1]
        pages = view.kv.shape[1]
        code = _dtype_code(q.dtype)
        if chunk:
            window = self._span(window, chunk)
        window = int(window or 0)         # (negative: chunks, see _span)
        if sinks is not None:
            # (float32 [heads]: exp(sink) of a query's head stands in its softmax's denominator)
            self._need(sinks, torch.float32, "sinks")
            if sinks.numel() != heads:
                raise KernelError("one sink per query head")
        keep_first = int(keep_first or 0) if window > 0 else 0
        tensor_cores = (self.tensor_core_attention
                        and self.lib.mlxone_attention_mma_supports(head_dim, code))
        if keep_first and not tensor_cores:
            self._call("mlxone_attention_generic_keep", _c_void_p(_ptr(q)), _c_void_p(_ptr(view.kv)),
                       _c_void_p(_ptr(view.block_table)), _c_int(width), _c_int(view.page_size),
                       _c_int(pages), _c_void_p(_ptr(ctx.positions)),
                       _c_void_p(_ptr(ctx.token_request)), _c_void_p(_ptr(out)), _c_int(tokens),
                       _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_float(scale),
                       _c_int(window), _c_int(keep_first), _c_int(code), _c_void_p(_ptr(sinks)),
                       _c_void_p(_ptr(self.error_flag)))
            return out
        if tensor_cores:
            if ctx.max_portion == 1 and tokens == ctx.requests:
                self._decode_attention(q, out, ctx.requests, heads, kv_heads, head_dim, scale,
                                       window, ctx, view, sinks, keep_first)
                return out
            # The decodes at the head of a mixed step go to the split-key kernel, which reads
            # each request's keys once for all its query heads; as one-token portions in the
            # prefill kernel they would each fill a tile of 64 or 128 query rows with one row.
            singles = min(getattr(ctx, "leading_single", 0), ctx.requests)
            if singles < self.split_singles_from:
                singles = 0
            if singles:
                self._decode_attention(q, out, singles, heads, kv_heads, head_dim, scale, window,
                                       ctx, view, sinks, keep_first)
            # the other requests: the tables, starts and histories from request ``singles`` on
            # (token numbers in request_start stay those of the whole step)
            rest = ctx.requests - singles
            table = view.block_table[singles:]
            starts, history = ctx.request_start[singles:], ctx.history[singles:]
            if (self.tcgen05_attention and q.dtype == torch.bfloat16
                    and self.lib.mlxone_attention_tcgen05_supports(
                        _c_int(head_dim), _c_int(heads), _c_int(kv_heads), _c_int(view.page_size))):
                # few query tiles (a prompt's portion beside a step's decodes): their keys are
                # cut into parts that run side by side, and a merge follows
                bound = min(ctx.max_context, width * view.page_size)
                if window:
                    bound = min(bound, abs(window) + ctx.max_portion + keep_first)
                splits = 1
                if self.prefill_key_splits:
                    splits = self.lib.mlxone_attention_tcgen05_splits(
                        _c_int(tokens - singles), _c_int(rest), _c_int(heads), _c_int(kv_heads),
                        _c_int(bound))
                partial = None
                if splits > 1:
                    partial = torch.empty(tokens * heads * splits * (head_dim + 2),
                                          dtype=torch.float32, device=self.device)
                self._call("mlxone_attention_prefill_tcgen05_keep", _c_void_p(_ptr(q)),
                           _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(table)),
                           _c_int(width), _c_int(view.page_size), _c_int(pages),
                           _c_void_p(_ptr(starts)), _c_void_p(_ptr(history)),
                           _c_void_p(_ptr(out)), _c_int(tokens), _c_int(rest),
                           _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_float(scale),
                           _c_int(window or 0), _c_int(keep_first), _c_int(splits),
                           _c_void_p(_ptr(partial)), _c_void_p(_ptr(sinks)),
                           _c_void_p(_ptr(self.error_flag)))
                if partial is not None:
                    # (the leading single tokens are the decode kernel's: their rows stay)
                    skip = singles * heads * splits * (head_dim + 2)
                    self._call("mlxone_attention_merge", _c_void_p(_ptr(partial[skip:])),
                               _c_void_p(_ptr(out[singles:])), _c_int((tokens - singles) * heads),
                               _c_int(splits), _c_int(head_dim))
            else:
                self._call("mlxone_attention_prefill_keep", _c_void_p(_ptr(q)),
                           _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(table)),
                           _c_int(width), _c_int(view.page_size), _c_int(pages),
                           _c_void_p(_ptr(starts)), _c_void_p(_ptr(history)),
                           _c_void_p(_ptr(out)), _c_int(tokens), _c_int(rest),
                           _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_float(scale),
                           _c_int(window or 0), _c_int(keep_first), _c_void_p(_ptr(sinks)))
            return out
        self._call("mlxone_attention_generic", _c_void_p(_ptr(q)), _c_void_p(_ptr(view.kv)),
                   _c_void_p(_ptr(view.block_table)), _c_int(width),
                   _c_int(view.page_size), _c_int(pages),
                   _c_void_p(_ptr(ctx.positions)), _c_void_p(_ptr(ctx.token_request)),
                   _c_void_p(_ptr(out)), _c_int(tokens), _c_int(heads), _c_int(kv_heads),
                   _c_int(head_dim), _c_float(scale), _c_int(window or 0),
                   _c_int(code), _c_void_p(_ptr(sinks)), _c_void_p(_ptr(self.error_flag)))
        return out

    def _decode_attention(self, q, out, requests, heads, kv_heads, head_dim, scale, window, ctx,
                          view, sinks=None, keep_first=0) -> None:
        """The split-key kernel for the first ``requests`` requests of the step, one token each
        (token i is request i's): rows 0 to requests - 1 of q, positions, table and out."""
        width = view.block_table.shape[1]
        splits, partial = self._decode_plan(requests, heads, kv_heads, head_dim, width, window,
                                            view, keep_first)
        if keep_first:
            self._call("mlxone_attention_decode_keep", _c_void_p(_ptr(q)), _c_void_p(_ptr(view.kv)),
                       _c_void_p(_ptr(view.block_table)), _c_int(width), _c_int(view.page_size),
                       _c_int(view.kv.shape[1]), _c_void_p(_ptr(ctx.positions)),
                       _c_void_p(_ptr(out)), _c_void_p(_ptr(partial)), _c_int(requests),
                       _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(splits),
                       _c_float(scale), _c_int(window), _c_int(keep_first), _c_void_p(_ptr(sinks)))
            if partial is not None:
                self.launches += 1          # the merge kernel
            return
        self._call("mlxone_attention_decode_sinks", _c_void_p(_ptr(q)), _c_void_p(_ptr(view.kv)),
                   _c_void_p(_ptr(view.block_table)), _c_int(width), _c_int(view.page_size),
                   _c_int(view.kv.shape[1]), _c_void_p(_ptr(ctx.positions)), _c_void_p(_ptr(out)),
                   _c_void_p(_ptr(partial)), _c_int(requests), _c_int(heads), _c_int(kv_heads),
                   _c_int(head_dim), _c_int(splits), _c_float(scale), _c_int(window or 0),
                   _c_void_p(_ptr(sinks)))
        if partial is not None:
            self.launches += 1          # the merge kernel

    def _decode_plan(self, requests, heads, kv_heads, head_dim, width, window, view, keep_first=0):
        """Key splits of a decode attention launch and the scratch for their partial results
        (None when a thread-block cluster merges them, or there is one split)."""
        splits = self.decode_splits(requests, heads, kv_heads, head_dim, width * view.page_size,
                                    window, keep_first)
        clustered = self.cluster_merge and splits <= min(self.cluster_merge_max_splits, 8)
        partial = None
        if splits > 1 and not clustered:
            partial = torch.empty(requests * heads * splits * (head_dim + 2),
                                  dtype=torch.float32, device=self.device)
        return splits, partial

    def decode_splits(self, requests: int, heads: int, kv_heads: int, head_dim: int,
                      context_bound: int, window: int | None, keep_first: int = 0) -> int:
        """Into how many parts the decode kernel cuts a request's keys: as many blocks as the
        GPU holds at once (one wave), but at least four tiles of 32 keys per part."""
        if window:
            context_bound = min(context_bound, abs(window) + 31 + (-(-keep_first // 32)) * 32)
        tiles = max(-(-context_bound // 32), 1)
        blocks_per_sm = self.lib.mlxone_attention_decode_resident(_c_int(head_dim))
        groups = kv_heads * (-(-(heads // kv_heads) // 8))
        wanted = max(self._sm_count * blocks_per_sm // max(requests * groups, 1), 1)
        return max(min(wanted, tiles // 4), 1)

    def argmax(self, logits):
        self._need(logits, torch.float32, "logits")
        rows, vocab = logits.shape
        out = torch.empty((rows,), dtype=torch.int32, device=self.device)
        scratch = self.lib.mlxone_argmax_scratch(rows, vocab)
        values = indices = None
        if scratch:
            values = torch.empty(scratch, dtype=torch.float32, device=self.device)
            indices = torch.empty(scratch, dtype=torch.int32, device=self.device)
        self._call("mlxone_argmax", _c_void_p(_ptr(logits)), _c_int(rows), _c_int(vocab),
                   _c_void_p(_ptr(out)), _c_void_p(_ptr(values)), _c_void_p(_ptr(indices)))
        return out

    def decode_advance(self, chosen, token_ids, positions, history, record, counter):
        """In place: token_ids = chosen, positions += 1, history += 1,
        record[counter] = chosen, counter += 1 (all int32 on the device)."""
        for tensor in (chosen, token_ids, positions, history, record, counter):
            self._need(tensor, torch.int32, "decode_advance argument")
        self._call("mlxone_decode_advance", _c_void_p(_ptr(chosen)), _c_void_p(_ptr(token_ids)),
                   _c_void_p(_ptr(positions)), _c_void_p(_ptr(history)), _c_void_p(_ptr(record)),
                   _c_void_p(_ptr(counter)), _c_int(chosen.numel()), _c_int(record.shape[0]))

    def publish_tokens(self, chosen, index, published):
        """published[index[i]] = chosen[i] (all int32 on the device). Returns the step's report
        for the host: the chosen tokens followed by the value of the kernels' error flag, so
        that one copy brings both."""
        report = torch.empty(chosen.numel() + 1, dtype=torch.int32, device=self.device)
        self._call("mlxone_publish_tokens", _c_void_p(_ptr(chosen)), _c_void_p(_ptr(index)),
                   _c_void_p(_ptr(published)), _c_int(chosen.numel()), _c_int(published.numel()),
                   _c_void_p(_ptr(report)), _c_void_p(_ptr(self.error_flag)))
        return report

    def resolve_tokens(self, token_ids, source, published):
        """token_ids[t] = published[source[t]] where source[t] >= 0, in place."""
        self._call("mlxone_resolve_tokens", _c_void_p(_ptr(token_ids)), _c_void_p(_ptr(source)),
                   _c_void_p(_ptr(published)), _c_int(token_ids.numel()),
                   _c_int(published.numel()))

    def reserve_sample_scratch(self, rows: int, vocab: int) -> None:
        """Makes the sampling kernel's scratch large enough for ``rows`` rows now, so that no
        call inside a graph capture has to allocate it."""
        scratch = self._sample_scratch
        if scratch is None or scratch.numel() < rows * vocab:
            self._sample_scratch = torch.empty(rows * vocab, dtype=torch.float32,
                                               device=self.device)

    def sample(self, logits, temperature, top_k, top_p, seed, step):
        """Per row: temperature (float32, > 0), top_k (int32, <= 0 = off), top_p (float32,
        >= 1 = off), seed (int64), step (int32). Returns (tokens int32, probabilities)."""
        self._need(logits, torch.float32, "logits")
        rows, vocab = logits.shape
        for tensor, dtype, what in ((temperature, torch.float32, "temperature"),
                                    (top_k, torch.int32, "top_k"), (top_p, torch.float32, "top_p"),
                                    (seed, torch.int64, "seed"), (step, torch.int32, "step")):
            self._need(tensor, dtype, what)
            if tensor.numel() != rows:
                raise KernelError(f"{what} must have one entry per row")
        scratch = self._sample_scratch
        if scratch is None or scratch.numel() < rows * vocab:
            scratch = torch.empty(rows * vocab, dtype=torch.float32, device=self.device)
            self._sample_scratch = scratch
        out = torch.empty((rows,), dtype=torch.int32, device=self.device)
        self._call("mlxone_sample", _c_void_p(_ptr(logits)), _c_int(rows), _c_int(vocab),
                   _c_void_p(_ptr(temperature)), _c_void_p(_ptr(top_k)), _c_void_p(_ptr(top_p)),
                   _c_void_p(_ptr(seed)), _c_void_p(_ptr(step)), _c_void_p(_ptr(scratch)),
                   _c_void_p(_ptr(out)))
        return out, scratch[: rows * vocab].view(rows, vocab)
