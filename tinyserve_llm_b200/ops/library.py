"""
Python face of the CUDA kernel library: loads the shared object (building it at first use) and
wraps each exported kernel launcher with argument checks.  There is no CPU fallback and no library
attention: if the shared object cannot be built or loaded, constructing `Ops` raises.
"""

from __future__ import annotations

import ctypes
import os

import torch

from tinyserve_llm_b200.ops.build import build_library

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    """A kernel launcher refused its arguments or the launch failed."""


# Argument types of the exported functions (p: pointer or stream, i: int, l: long long, f: float), set once
# on the ctypes functions so that a call converts plain Python numbers itself: at some hundred launches
# a step, wrapper objects per argument were a tenth of an eager step's host time.
_SIGNATURES = {
    "ts_silu_mul": ("int", "ppiiip"),
    "ts_attention_bf16_scratch_floats": ("long long", "iiii"),
    "ts_attention_bf16_supported": ("int", "iiii"),
    "ts_paged_attention_bf16": ("int", "pppplliipippiiiiiiifiplpip"),
    "ts_paged_attention_generic": ("int", "pppplliipippiiiifiip"),
    "ts_attention_tcgen05_supported": ("int", "iiiii"),
    "ts_prefill_attention_tcgen05": ("int", "ppppiiiipippiiiiiifpipp"),
    "ts_embedding": ("int", "pppiiiip"),
    "ts_feed_tokens": ("int", "pipip"),
    "ts_gemm_tcgen05_supported": ("int", "ppiiil"),
    "ts_gemm_tcgen05": ("int", "pppiiilliipp"),
    "ts_gemm_tcgen05_set_pairing": ("void", "i"),
    "ts_last_error": ("const char*", ""),
    "ts_abi_version": ("int", ""),
    "ts_set_chaining": ("void", "i"),
    "ts_add_rmsnorm": ("int", "ppppppiifiipip"),
    "ts_copy_page_slots": ("int", "ppiiiiiiiiip"),
    "ts_rope_store": ("int", "ppppiipipplliiiiiiiip"),
    "ts_sample_scratch_words": ("int", "ii"),
    "ts_sample": ("int", "plpppiipip"),
    "ts_sgemm_nt": ("int", "pppiiilllp"),
    "ts_skinny_linear_max_rows": ("int", ""),
    "ts_skinny_linear": ("int", "pppiiilliip"),
    "ts_skinny_qkv_rope_store": ("int", "pppiilpppiipipplliiiiiip"),
}
_CTYPES = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_longlong, "f": ctypes.c_float}
_RETURNS = {"int": ctypes.c_int, "long long": ctypes.c_longlong, "void": None, "const char*": ctypes.c_char_p}

# Where a bounded wait inside a kernel gave up, by the code it left in the error word.
_WAIT_CODES: dict[int, tuple[str, str]] = {
    1: ("gemm_tcgen05", "TMA producer waiting for a free ring slot"),
    2: ("gemm_tcgen05", "MMA issuer waiting for operands"),
    3: ("gemm_tcgen05", "epilogue waiting for an accumulator"),
    4: ("gemm_tcgen05", "MMA issuer waiting for a drained accumulator"),
    11: ("attention_tcgen05", "loader waiting for a free key/value stage"),
    12: ("attention_tcgen05", "MMA issuer waiting for the query tile"),
    13: ("attention_tcgen05", "MMA issuer waiting for a key/value tile"),
    14: ("attention_tcgen05", "MMA issuer waiting for the softmax's probabilities"),
    15: ("attention_tcgen05", "softmax waiting for scores"),
    16: ("attention_tcgen05", "epilogue waiting for the last product"),
    17: ("attention_tcgen05", "softmax waiting for the previous product before rescaling"),
}


def register_kernel(name: str, returns: str, arguments: str) -> None:
    """
    Declares an exported launcher that `Ops.call(name, ...)` may call: `returns` is one of "int"
    (0 = success, the library's error text otherwise), "long long", "void", "const char*";
    `arguments` one letter per argument (p: pointer or stream, i: int, l: long long, f: float).
    A part that brings a kernel of its own (a .cu file beside the others, or an extension it loads
    with `Ops.load_extension`) registers it here, from its own module; nothing in this file changes.
    """
    if returns not in _RETURNS or any(a not in _CTYPES for a in arguments):
        raise ValueError(f"register_kernel({name!r}): unknown return type or argument letter")
    _SIGNATURES[name] = (returns, arguments)
    if _OPS is not None:
        _OPS._bind(name)


def register_wait_codes(kernel: str, codes: dict[int, str]) -> None:
    """Names the codes a kernel's bounded waits leave in the error word (see `Ops.error_word`)."""
    for code, where in codes.items():
        if code in _WAIT_CODES and _WAIT_CODES[code][0] != kernel:
            raise ValueError(f"wait code {code} belongs to {_WAIT_CODES[code][0]} already")
        _WAIT_CODES[code] = (kernel, where)


def _ptr(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch, so by the short way where torch has one."""
    if _RAW_STREAM is not None and _RAW_DEVICE is not None:
        return _RAW_STREAM(_RAW_DEVICE())
    return torch.cuda.current_stream().cuda_stream


class Ops:
    """One instance per process is enough; see `get_ops()`."""

    def __init__(self, lib_path: str | None = None) -> None:
        self.lib_path = lib_path or build_library()
        try:
            self.lib = ctypes.CDLL(self.lib_path)
        except OSError as exc:
            raise KernelError(f"cannot load the CUDA kernel library {self.lib_path}: {exc}") from None
        self._functions: dict[str, object] = {}       # launcher name -> (ctypes function, library it came from)
        self._extensions: dict[str, ctypes.CDLL] = {}
        for name in _SIGNATURES:
            self._bind(name)
        self.launches = 0            # kernels of this library launched (or captured into a graph) so far
        self.calls: dict[str, int] = {}   # calls per exported launcher (and "library_mm": products left to cuBLAS)
        self._error_word: torch.Tensor | None = None
        self.skinny_max_rows = int(self.lib.ts_skinny_linear_max_rows())
        # TINYSERVE_B200_CHAINING=0 launches every kernel fully serialised (no programmatic dependent launch)
        self.set_chaining(os.environ.get("TINYSERVE_B200_CHAINING", "1") != "0")
        # TINYSERVE_B200_PREFILL=mma keeps prompt attention on the mma.sync kernel (the tcgen05 one is the default)
        self.tcgen05_attention = os.environ.get("TINYSERVE_B200_PREFILL", "tcgen05") != "mma"
        # From this many rows of x the gate/up product runs on the engine's tcgen05 kernel with SwiGLU in its
        # epilogue: measured on a B200 against the library product plus an activation kernel, it is 8 to 13 % faster
        # from 512 rows on with Llama 3.2 1B's sizes (3B and 3.1 8B: the same or faster), and slower between 257 and
        # about 450 rows, where three row tiles fit the SMs badly.
        self.tcgen05_swiglu_min_rows = int(os.environ.get("TINYSERVE_B200_SWIGLU_ROWS", "512"))
        # up to this many rows the gate/up product with SwiGLU runs on the decode product (measured on a B200 with Llama
        # 3.2 1B's sizes, whole decode steps: 4 to 6 % faster than the library product plus the activation kernel at 12,
        # 16, 24 and 32 rows, since the weights go through the cp.async ring)
        self.swiglu_skinny_rows = self.skinny_max_rows

    def set_chaining(self, enabled: bool) -> None:
        self.chaining = bool(enabled)
        self.lib.ts_set_chaining(1 if enabled else 0)

    # ------------------------------------------------------------------ helpers
    def _bind(self, name: str, lib: ctypes.CDLL | None = None) -> None:
        returns, arguments = _SIGNATURES[name]
        owner = None
        for candidate in ([lib] if lib is not None else [self.lib, *self._extensions.values()]):
            if hasattr(candidate, name):
                owner = candidate
                break
        if owner is None:
            raise KernelError(f"the CUDA kernel library {self.lib_path} does not export {name}")
        fn = getattr(owner, name)
        fn.restype = _RETURNS[returns]
        fn.argtypes = [_CTYPES[a] for a in arguments]
        self._functions[name] = (fn, owner)

    def _call(self, name: str, *args) -> None:
        fn, owner = self._functions[name]
        if fn(*args) != 0:
            raise KernelError(owner.ts_last_error().decode())
        self.launches += 1
        self.calls[name] = self.calls.get(name, 0) + 1

    def call(self, name: str, *args):
        """
        Calls a registered launcher (`register_kernel`) with plain numbers and `data_ptr()`s.  An
        "int" launcher is a kernel launch: nonzero raises KernelError with the library's text, and
        the launch is counted.  Other return types hand back their value.
        """
        if name not in self._functions:
            if name not in _SIGNATURES:
                raise KernelError(f"{name} is not a registered kernel launcher; call register_kernel first")
            self._bind(name)
        if _SIGNATURES[name][0] == "int":
            return self._call(name, *args)
        return self._functions[name][0](*args)

    @staticmethod
    def stream() -> int:
        """The current CUDA stream's handle, as launchers take it."""
        return _stream()

    def error_word(self) -> torch.Tensor:
        """
        One int32 in pinned host memory that kernels with bounded waits write a code into when a
        wait runs out (its `data_ptr()` is what their launchers take).  `check_device_errors` reads
        it before every step and names the kernel by the registered code (`register_wait_codes`).
        """
        if self._error_word is None:
            self._error_word = torch.zeros((1,), dtype=torch.int32).pin_memory()
        return self._error_word

    def load_extension(self, name: str, sources: list[str], kernels: dict[str, tuple[str, str]]) -> None:
        """
        Compiles a part's own .cu files for sm_100a into a shared library of their own (they may
        include this library's common.cuh and report errors the same way), loads it and registers
        its launchers: `kernels` maps an exported name to (returns, arguments) as `register_kernel`
        takes them.  Done once per name and process.
        """
        if name in self._extensions:
            return
        from tinyserve_llm_b200.ops.build import build_extension
        path = build_extension(name, sources)
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:
            raise KernelError(f"cannot load the kernel extension {path}: {exc}") from None
        lib.ts_last_error.restype = ctypes.c_char_p
        self._extensions[name] = lib
        for kernel, (returns, arguments) in kernels.items():
            register_kernel(kernel, returns, arguments)
            self._bind(kernel, lib)

    @staticmethod
    def _check(t: torch.Tensor, name: str, dtype: torch.dtype | tuple | None = None, dims: int | None = None) -> None:
        if not t.is_cuda:
            raise KernelError(f"{name} must be a CUDA tensor; the engine has no CPU path")
        if not t.is_contiguous():
            raise KernelError(f"{name} must be contiguous")
        if dtype is not None:
            allowed = dtype if isinstance(dtype, tuple) else (dtype,)
            if t.dtype not in allowed:
                raise KernelError(f"{name} has dtype {t.dtype}, expected one of {allowed}")
        if dims is not None and t.dim() != dims:
            raise KernelError(f"{name} has {t.dim()} dimensions, expected {dims}")

    # ------------------------------------------------------------------ kernels
    def embedding(self, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        self._check(table, "embedding table", tuple(_DTYPE_CODE), 2)
        self._check(ids, "token ids", torch.int32, 1)
        out = torch.empty((ids.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
        self._call("ts_embedding", _ptr(table), _ptr(ids), _ptr(out), ids.shape[0], table.shape[1],
                   table.shape[0], _DTYPE_CODE[table.dtype], _stream())
        return out

    def feed_tokens(self, ids: torch.Tensor, source: torch.Tensor) -> None:
        """In place: an id slot that holds -(j + 2) becomes source[j] (the previous step's sample j, still on the device)."""
        self._check(ids, "token ids", torch.int32, 1)
        self._check(source, "sampled tokens", torch.int32, 1)
        self._call("ts_feed_tokens", _ptr(ids), ids.shape[0], _ptr(source), source.shape[0], _stream())

    def add_rmsnorm(self, x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, eps: float,
                    rows: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """
        (normalised, residual stream).  Without `rows`, both results overwrite their inputs (x and
        residual) and x starts the stream when residual is None.  With `rows` (int32 row indices)
        only those rows are normalised into a new compact tensor and the stream is not written.
        """
        self._check(x, "x", tuple(_DTYPE_CODE), 2)
        self._check(weight, "norm weight", tuple(_DTYPE_CODE), 1)
        hidden = x.shape[1]
        if weight.shape[0] != hidden:
            raise KernelError(f"norm weight has {weight.shape[0]} elements for rows of {hidden}")
        if residual is not None:
            self._check(residual, "residual", x.dtype, 2)
            if residual.shape != x.shape:
                raise KernelError(f"residual {tuple(residual.shape)} does not match x {tuple(x.shape)}")
        if rows is None:
            if residual is None:
                out = torch.empty_like(x)
                new_residual, residual_out = x, None
            else:
                out, new_residual, residual_out = x, residual, residual
            count = x.shape[0]
        else:
            self._check(rows, "rows", torch.int32, 1)
            count = rows.shape[0]
            out = torch.empty((count, hidden), dtype=x.dtype, device=x.device)
            new_residual, residual_out = residual, None
        self._call("ts_add_rmsnorm", _ptr(x), _ptr(residual), _ptr(weight), _ptr(out), _ptr(residual_out), _ptr(rows),
                   count, hidden, eps, _DTYPE_CODE[x.dtype],
                   _DTYPE_CODE[weight.dtype], 0, 0, _stream())
        return out, new_residual

    def embed_rmsnorm(self, table: torch.Tensor, ids: torch.Tensor, weight: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
        """
        (normalised, residual stream) of the model's first norm with the token embedding read straight
        into it: row t of the stream is table[ids[t]] (zeros for an id outside the table), one kernel
        instead of a gather and a norm.
        """
        self._check(table, "embedding table", tuple(_DTYPE_CODE), 2)
        self._check(ids, "token ids", torch.int32, 1)
        self._check(weight, "norm weight", tuple(_DTYPE_CODE), 1)
        hidden = table.shape[1]
        if weight.shape[0] != hidden:
            raise KernelError(f"norm weight has {weight.shape[0]} elements for rows of {hidden}")
        out = torch.empty((ids.shape[0], hidden), dtype=table.dtype, device=table.device)
        stream = torch.empty_like(out)
        self._call("ts_add_rmsnorm", _ptr(table), 0, _ptr(weight), _ptr(out), _ptr(stream), 0, ids.shape[0], hidden, eps,
                   _DTYPE_CODE[table.dtype], _DTYPE_CODE[weight.dtype], _ptr(ids), table.shape[0], _stream())
        return out, stream

    def rope_store(self, qkv: torch.Tensor, ctx, binding, table: torch.Tensor | None, nh: int, nkv: int, hd: int) -> None:
        self._check(qkv, "qkv", tuple(_DTYPE_CODE), 2)
        if qkv.shape[1] != (nh + 2 * nkv) * hd:
            raise KernelError(f"qkv rows have {qkv.shape[1]} columns, expected {(nh + 2 * nkv) * hd}")
        if binding.k_pool.dtype != qkv.dtype:
            raise KernelError(f"cache pool is {binding.k_pool.dtype} but activations are {qkv.dtype}")
        rot, rows = 0, 0
        if table is not None:
            self._check(table, "rotary table", torch.float32, 2)
            rows, rot = table.shape
        self._call("ts_rope_store", _ptr(qkv), _ptr(ctx.positions), _ptr(ctx.seq_of_token), _ptr(table), rows,
                   rot, _ptr(binding.block_table), binding.table_width, _ptr(binding.k_pool),
                   _ptr(binding.v_pool), binding.page_stride, binding.entry_offset,
                   binding.page_tokens, binding.num_pages, qkv.shape[0], nh, nkv,
                   hd, 1 if binding.writes else 0, _DTYPE_CODE[qkv.dtype], _stream())

    def linear_rope_store(self, x: torch.Tensor, weight: torch.Tensor, ctx, binding, table: torch.Tensor | None,
                          nh: int, nkv: int, hd: int) -> torch.Tensor | None:
        """
        The q/k/v projection of a step of a few tokens with the rotation and the cache write in its
        epilogue: returns qkv [T, (nh + 2 nkv) * hd] whose q columns are rotated (k and v are in
        the cache only), or None where the fused kernel does not take the case (then: `linear`,
        `rope_store`).  Takes bfloat16, as many tokens as the decode product does, a rotary width equal to the head size.
        """
        if (not self._skinny(x, weight) or hd % 16 or binding.k_pool.dtype != torch.bfloat16
                or binding.block_table is None or (table is not None and table.shape[1] != hd)):
            return None
        self._check(x, "x", torch.bfloat16, 2)
        self._check(weight, "weight", torch.bfloat16, 2)
        if tuple(weight.shape) != ((nh + 2 * nkv) * hd, x.shape[1]):
            raise KernelError(f"linear_rope_store: weight is {tuple(weight.shape)}, expected {((nh + 2 * nkv) * hd, x.shape[1])}")
        rows = 0
        if table is not None:
            self._check(table, "rotary table", torch.float32, 2)
            rows = table.shape[0]
        qkv = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16, device=x.device)
        self._call("ts_skinny_qkv_rope_store", _ptr(weight), _ptr(x), _ptr(qkv), x.shape[0], x.shape[1],
                   x.stride(0), _ptr(ctx.positions), _ptr(ctx.seq_of_token), _ptr(table), rows,
                   hd, _ptr(binding.block_table), binding.table_width, _ptr(binding.k_pool),
                   _ptr(binding.v_pool), binding.page_stride, binding.entry_offset,
                   binding.page_tokens, binding.num_pages, nh, nkv, hd,
                   1 if binding.writes else 0, _stream())
        return qkv

    def paged_attention(self, qkv: torch.Tensor, ctx, binding, nh: int, nkv: int, hd: int, scale: float,
                        window: int, generic: bool = False) -> torch.Tensor:
        """
        [T, nh * hd].  bfloat16 with head size 64 or 128 and pages of a multiple of 64 tokens runs on
        the tensor-core kernels (prefill tiles and split-key decode); everything else, and
        `generic=True`, on the generic kernel.
        """
        self._check(qkv, "qkv", tuple(_DTYPE_CODE), 2)
        out = torch.empty((qkv.shape[0], nh * hd), dtype=qkv.dtype, device=qkv.device)
        if (not generic and qkv.dtype == torch.bfloat16 and getattr(ctx, "cu_q", None) is not None
                and self.lib.ts_attention_bf16_supported(hd, binding.page_tokens, nh, nkv)):
            num_seqs = ctx.ctx_lens.shape[0]
            scratch, floats = None, 0
            max_q_len = ctx.max_q_len
            prefill_seqs = getattr(ctx, "prefill_seqs", None)      # the step runner lists them; a bare context may not
            num_prefill = prefill_seqs.shape[0] if prefill_seqs is not None else 0
            if (max_q_len > 1 and self.tcgen05_attention and self.lib.ts_attention_tcgen05_supported(
                    hd, binding.page_tokens, nh, nkv, window)):
                # prompt portions on the tcgen05 kernel; requests that feed one token stay with the split-key kernels
                per_entry = nkv * binding.page_tokens * hd
                self._call("ts_prefill_attention_tcgen05", _ptr(qkv), _ptr(out), _ptr(binding.k_pool), _ptr(binding.v_pool),
                           binding.num_pages, binding.page_stride // per_entry,
                           binding.entry_offset // per_entry, binding.page_tokens, _ptr(binding.block_table),
                           binding.table_width, _ptr(ctx.cu_q), _ptr(ctx.ctx_lens), num_seqs,
                           qkv.shape[0], max_q_len, nh, nkv, hd, scale,
                           _ptr(prefill_seqs), num_prefill, self.error_word().data_ptr(), _stream())
                if ctx.min_q_len > 1:
                    return out
                max_q_len = 1
            # the decode grid and scratch follow the longest request that feeds ONE token: a long prompt portion beside
            # short decodes must not size them (a bare context may not say, then the longest request of all does)
            decode_ctx = getattr(ctx, "max_decode_ctx_len", ctx.max_ctx_len)
            if ctx.min_q_len <= 1:
                floats = self.lib.ts_attention_bf16_scratch_floats(num_seqs, nh, hd,
                                                                   decode_ctx)
                key = ("attention", floats)
                scratch = ctx.scratch.get(key)
                if scratch is None:
                    scratch = ctx.scratch[key] = torch.empty((floats,), dtype=torch.float32, device=qkv.device)
            self._call("ts_paged_attention_bf16", _ptr(qkv), _ptr(out), _ptr(binding.k_pool), _ptr(binding.v_pool),
                       binding.page_stride, binding.entry_offset, binding.page_tokens,
                       binding.num_pages, _ptr(binding.block_table), binding.table_width,
                       _ptr(ctx.cu_q), _ptr(ctx.ctx_lens), num_seqs, max_q_len,
                       min(ctx.min_q_len, max_q_len), decode_ctx, nh, nkv, hd,
                       scale, window, _ptr(scratch), floats, _ptr(prefill_seqs),
                       num_prefill, _stream())
            if ctx.min_q_len <= 1:
                self.launches += 1 if max_q_len <= 1 else 2          # decode + combine (+ prefill) in one call
            return out
        self._call("ts_paged_attention_generic", _ptr(qkv), _ptr(out), _ptr(binding.k_pool), _ptr(binding.v_pool),
                   binding.page_stride, binding.entry_offset, binding.page_tokens,
                   binding.num_pages, _ptr(binding.block_table), binding.table_width,
                   _ptr(ctx.positions), _ptr(ctx.seq_of_token), qkv.shape[0], nh, nkv, hd,
                   scale, window, _DTYPE_CODE[qkv.dtype], _stream())
        return out

    def silu_mul(self, gate_up: torch.Tensor) -> torch.Tensor:
        self._check(gate_up, "gate_up", tuple(_DTYPE_CODE), 2)
        if gate_up.shape[1] % 2:
            raise KernelError("gate_up rows must hold gate and up halves of equal width")
        inter = gate_up.shape[1] // 2
        out = torch.empty((gate_up.shape[0], inter), dtype=gate_up.dtype, device=gate_up.device)
        self._call("ts_silu_mul", _ptr(gate_up), _ptr(out), gate_up.shape[0], inter,
                   _DTYPE_CODE[gate_up.dtype], _stream())
        return out

    def linear(self, x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None,
               out: torch.Tensor | None = None) -> torch.Tensor:
        """
        x [M, K] . weight[N, K]^T.  float32: the engine's FFMA kernel.  bfloat16: up to 32 rows of x on
        the engine's weight-streaming kernel, more on the library product (cuBLAS through torch.mm).
        `out` (contiguous [M, N] of the output dtype) receives the product instead of a new tensor.
        """
        self._check(x, "x", tuple(_DTYPE_CODE), 2)
        self._check(weight, "weight", x.dtype, 2)
        if x.shape[1] != weight.shape[1]:
            raise KernelError(f"linear: x has {x.shape[1]} columns, the weight {weight.shape[1]}")
        out_dtype = out_dtype or x.dtype
        if x.dtype == torch.float32 and out_dtype != torch.float32:
            raise KernelError("linear: the float32 product has float32 output")
        if out is None:
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
        else:
            self._check(out, "out", out_dtype, 2)
            if tuple(out.shape) != (x.shape[0], weight.shape[0]):
                raise KernelError(f"linear: out is {tuple(out.shape)}, the product {(x.shape[0], weight.shape[0])}")
        if x.dtype == torch.float32:
            self._call("ts_sgemm_nt", _ptr(x), _ptr(weight), _ptr(out), x.shape[0], weight.shape[0],
                       x.shape[1], x.shape[1], weight.shape[1],
                       weight.shape[0], _stream())
            return out
        if self._skinny(x, weight):
            self._call("ts_skinny_linear", _ptr(weight), _ptr(x), _ptr(out), x.shape[0], weight.shape[0],
                       x.shape[1], x.shape[1], weight.shape[0], 0,
                       _DTYPE_CODE[out_dtype], _stream())
            if out_dtype == torch.float32:
                self.calls["ts_skinny_linear:float32_out"] = self.calls.get("ts_skinny_linear:float32_out", 0) + 1
            return out
        self.calls["library_mm"] = self.calls.get("library_mm", 0) + 1
        if out_dtype != x.dtype:
            return torch.mm(x, weight.t(), out_dtype=out_dtype, out=out)
        return torch.mm(x, weight.t(), out=out)

    def gemm_tcgen05(self, x: torch.Tensor, weight: torch.Tensor, *, swiglu: bool = False,
                     out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """
        x [M, K] . weight[N, K]^T on tcgen05 tensor cores with TMA-fed shared memory; `swiglu` stores
        silu(gate) * up of the two halves of the weight's rows instead ([M, N / 2]).
        """
        self._check(x, "x", torch.bfloat16, 2)
        self._check(weight, "weight", torch.bfloat16, 2)
        M, K = x.shape
        N = weight.shape[0]
        if weight.shape[1] != K:
            raise KernelError(f"gemm_tcgen05: x has {K} columns, the weight {weight.shape[1]}")
        out_dtype = out_dtype or torch.bfloat16
        cols = N // 2 if swiglu else N
        out = torch.empty((M, cols), dtype=out_dtype, device=x.device)
        if M == 0:
            return out
        self._call("ts_gemm_tcgen05", _ptr(weight), _ptr(x), _ptr(out), M, N, K, K,
                   cols, 1 if swiglu else 0, _DTYPE_CODE[out_dtype],
                   self.error_word().data_ptr(), _stream())
        return out

    def check_device_errors(self) -> None:
        """Raises if a kernel's bounded wait ran out (the word lives in pinned host memory: no sync needed)."""
        if self._error_word is not None and int(self._error_word[0]) != 0:
            code = int(self._error_word[0])
            self._error_word[0] = 0
            kernel, where = _WAIT_CODES.get(code, ("a kernel", "an unregistered wait"))
            raise KernelError(f"{kernel}: a bounded wait ran out of time ({where}; code {code})")

    def _skinny(self, x: torch.Tensor, weight: torch.Tensor) -> bool:
        """A few rows of bfloat16 x (a decode step): the engine's own weight-streaming kernel takes them."""
        return (x.dtype == torch.bfloat16 and 0 < x.shape[0] <= self.skinny_max_rows and x.shape[1] % 32 == 0
                and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)

    def linear_swiglu(self, x: torch.Tensor, gate_up_weight: torch.Tensor) -> torch.Tensor:
        """silu(x . Wgate^T) * (x . Wup^T) with Wgate, Wup the two halves of the weight's rows: [M, I]."""
        self._check(x, "x", tuple(_DTYPE_CODE), 2)
        self._check(gate_up_weight, "weight", x.dtype, 2)
        if gate_up_weight.shape[0] % 2 or x.shape[1] != gate_up_weight.shape[1]:
            raise KernelError("linear_swiglu: the weight must hold gate and up halves over x's columns")
        if not (self._skinny(x, gate_up_weight) and x.shape[0] <= self.swiglu_skinny_rows):
            if x.dtype == torch.bfloat16 and x.shape[0] >= self.tcgen05_swiglu_min_rows and self.lib.ts_gemm_tcgen05_supported(
                    _ptr(gate_up_weight), _ptr(x), x.shape[0], gate_up_weight.shape[0], x.shape[1],
                    x.shape[1]):
                # tcgen05 product with the activation in its epilogue: the [M, 2I] product never reaches memory
                return self.gemm_tcgen05(x, gate_up_weight, swiglu=True)
            return self.silu_mul(self.linear(x, gate_up_weight))
        inter = gate_up_weight.shape[0] // 2
        out = torch.empty((x.shape[0], inter), dtype=x.dtype, device=x.device)
        self._call("ts_skinny_linear", _ptr(gate_up_weight), _ptr(x), _ptr(out), x.shape[0],
                   gate_up_weight.shape[0], x.shape[1], x.shape[1], inter,
                   1, _DTYPE_CODE[x.dtype], _stream())
        return out

    def sample(self, logits: torch.Tensor, temperatures: torch.Tensor, keys: torch.Tensor) -> torch.Tensor:
        """int32 [rows]: greedy where temperature is 0, else a draw keyed by keys[row] (two uint32 as int32)."""
        self._check(logits, "logits", torch.float32, 2)
        self._check(temperatures, "temperatures", torch.float32, 1)
        self._check(keys, "keys", torch.int32, 2)
        rows = logits.shape[0]
        if temperatures.shape[0] != rows or tuple(keys.shape) != (rows, 2):
            raise KernelError("sample: one temperature and one key pair per logits row are needed")
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
        words = int(self.lib.ts_sample_scratch_words(rows, logits.shape[1]))
        scratch = torch.empty((max(words, 1),), dtype=torch.int32, device=logits.device)    # the chunks' best (value, index)
        self._call("ts_sample", _ptr(logits), logits.shape[1], _ptr(temperatures), _ptr(keys), _ptr(out),
                   rows, logits.shape[1], _ptr(scratch), words, _stream())
        self.launches += 1                                   # two kernels in one call
        return out

    def copy_page_slots(self, k_pool: torch.Tensor, v_pool: torch.Tensor, src: int, dst: int, num_slots: int) -> None:
        """Pools are [pages, entries, kv_heads, page_tokens, head_dim]."""
        self._check(k_pool, "k_pool", tuple(_DTYPE_CODE), 5)
        pages, entries, nkv, page_tokens, hd = k_pool.shape
        self._call("ts_copy_page_slots", _ptr(k_pool), _ptr(v_pool), pages, entries, nkv,
                   page_tokens, hd, k_pool.dtype.itemsize, src, dst,
                   num_slots, _stream())


_OPS: Ops | None = None


def get_ops() -> Ops:
    global _OPS
    if _OPS is None:
        _OPS = Ops()
    return _OPS
