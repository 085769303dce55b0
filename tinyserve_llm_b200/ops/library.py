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
    "ts_paged_attention_bf16_sigmoid": ("int", "pl" "ppp" "lliipippiiiiiiifiplpi" "pppl" "p"),
    "ts_paged_attention_bf16_masked": ("int", "pl" "ppp" "lllliipippiiiiiiifiifi" "plpi" "p"),
    "ts_attention_tcgen05_supported": ("int", "iiiii"),
    "ts_prefill_attention_tcgen05_dense": ("int", "pl" "ppp" "lpppiiiiiifpipp"),
    "ts_prefill_attention_tcgen05_masked": ("int", "pl" "ppp" "iiiipippiiiiiifiifi" "pipp"),
    "ts_prefill_attention_tcgen05": ("int", "ppppiiiipippiiiiiifpipp"),
    "ts_prefill_attention_tcgen05_sigmoid": ("int", "pl" "ppp" "iiiipippiiiiiifi" "pppl" "pipp"),
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
    "ts_skinny_linear_gated": ("int", "pppiiilliffp"),
    "ts_skinny_linear_unary": ("int", "pppiiilliffip"),
    "ts_gemm_tcgen05_gated": ("int", "pppiiilliffpp"),
    "ts_stream_norm": ("int", "ppppppiifppifiipppp"),
    "ts_linear_recurrence": ("int", "ppplllplppfffpipppiplpiiiipip"),
    "ts_head_norm_gate": ("int", "piplpippliiififip"),
    "ts_latent_prepare": ("int", "pliiippfppppplliipiiiip"),
    "ts_latent_attention": ("int", "pllpliipplliipipppiiiifiiplip"),
    "ts_latent_attention_scratch_floats": ("long long", "iiii"),
    "ts_set_latent_mma": ("void", "i"),
    "ts_moe_route": ("int", "ppppppiiiip"),
    "ts_moe_arrange": ("int", "ppppppiip"),
    "ts_moe_linear": ("int", "plpipipiipiiiffpiip"),
    "ts_moe_combine": ("int", "pppppiiiippp"),
    "ts_moe_route_grouped": ("int", "pppppppiiiiiiffp"),
    "ts_paged_attention_scored": ("int", "plpppllllii" "pippiiiiifiiipppl" "fiii" "p"),
    "ts_mingru_scan": ("int", "pliiiippppiplpiiiip"),
    "ts_unary_activation_rows": ("int", "ppliffip"),
    "ts_gated_activation": ("int", "ppiiiffip"),
    "ts_sgemm_nt_batched": ("int", "pppiiilllilllp"),
    "ts_qk_norm_rope_store": ("int", "pliiipppppfpifpppppllllii" "piiiiiiiiifiip"),
    "ts_sigmoid_gate": ("int", "plplpliifip"),
    "ts_paged_attention_split": ("int", "plpppllllii" "pippiiiiifiip"),
    "ts_short_conv_silu": ("int", "plppppiplpiiiip"),
    "ts_recurrence_scan": ("int", "ppliipppiplpiiiip"),
    "ts_delta_prepare": ("int", "pplppppl" "ppiiiiffip"),
    "ts_mlstm_prepare": ("int", "ppllpplppffppiplpppiiiip"),
    "ts_row_scaled_activation": ("int", "ppppiiiip"),
    "ts_difference_head_norm": ("int", "plipl" "piiii" "fffip"),
    "ts_scale_tanh_cap": ("int", "plffp"),
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
        # TINYSERVE_B200_LATENT=ffma keeps attention over a cached latent off the tensor-core kernel
        self.lib.ts_set_latent_mma(0 if os.environ.get("TINYSERVE_B200_LATENT", "mma") == "ffma" else 1)
        # From this many rows of x the gate/up product runs on the engine's tcgen05 kernel with SwiGLU in its
        # epilogue: measured on a B200 against the library product plus an activation kernel, it is 8 to 13 % faster
        # from 512 rows on with Llama 3.2 1B's sizes (3B and 3.1 8B: the same or faster), and slower between 257 and
        # about 450 rows, where three row tiles fit the SMs badly.
        self.tcgen05_swiglu_min_rows = int(os.environ.get("TINYSERVE_B200_SWIGLU_ROWS", "512"))
        # up to this many rows the gate/up product with SwiGLU runs on the decode product (measured on a B200 with Llama
        # 3.2 1B's sizes, whole decode steps: 4 to 6 % faster than the library product plus the activation kernel at 12,
        # 16, 24 and 32 rows, since the weights go through the cp.async ring)
        self.swiglu_skinny_rows = self.skinny_max_rows
        # from this many (token, expert) pairs a routed feed-forward's bfloat16 products go to the library's grouped product
        self.grouped_mm_min_pairs = int(os.environ.get("TINYSERVE_B200_GROUPED_PAIRS", "256"))

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
    def _check_rows(t: torch.Tensor, name: str) -> None:
        """[rows, columns] of an activation dtype on the device whose rows may be stretches of wider rows."""
        if not t.is_cuda or t.dtype not in _DTYPE_CODE or t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
            raise KernelError(f"{name} must be a [rows, columns] stretch of an activation dtype on the device")

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

    # ------------------------------------------------------------------ float32 residual stream
    def stream_norm(self, branch: torch.Tensor | None, w_close: torch.Tensor | None, stream: torch.Tensor,
                    w_open: torch.Tensor | None, eps: float, dtype: torch.dtype, rows: torch.Tensor | None = None,
                    table: torch.Tensor | None = None, ids: torch.Tensor | None = None, scale: float = 1.0,
                    centered: bool = False, plain_add: bool = False, positions: torch.Tensor | None = None,
                    position_frequencies: torch.Tensor | None = None, w_start: torch.Tensor | None = None) -> torch.Tensor | None:
        """
        stream (float32, in place) += closing norm of `branch` (if given; with `plain_add` the branch as
        it is); returns the opening norm of the sum in `dtype` (if `w_open` is given; with `centered` a
        layer norm without bias instead of an RMS norm).  With `rows` only those rows are normed, into a
        compact output, and the stream is left as it is.  With `table` and `ids` the rows
        table[ids] * scale start the stream instead, plus, with `positions` and `position_frequencies` (float32
        [ceil(width / 2)]), the vector whose entry 2i is sin(position * frequency i) and entry 2i + 1 its cosine;
        with `w_start` the gathered rows are normed with that weight (as the opening norm norms: RMS, or centered)
        before they start the stream.  Weights are float32 and multiply as given.
        """
        self._check(stream, "residual stream", torch.float32, 2)
        width = stream.shape[1]
        if w_start is not None and ids is None:
            raise KernelError("stream_norm: a norm on the embedding rows needs token ids")
        for w, name in ((w_close, "closing weight"), (w_open, "opening weight"), (w_start, "embedding norm weight")):
            if w is not None:
                self._check(w, name, torch.float32, 1)
                if w.shape[0] != width:
                    raise KernelError(f"{name} has {w.shape[0]} elements for rows of {width}")
        if branch is not None:
            self._check(branch, "branch", dtype, 2)
            if branch.shape != stream.shape:
                raise KernelError(f"branch {tuple(branch.shape)} does not match the stream {tuple(stream.shape)}")
        if ids is not None:
            self._check(table, "embedding table", dtype, 2)
            self._check(ids, "token ids", torch.int32, 1)
            if table.shape[1] != width or ids.shape[0] != stream.shape[0]:
                raise KernelError("stream_norm: the table's rows or the number of ids do not match the stream")
        if position_frequencies is not None:
            self._check(position_frequencies, "position frequencies", torch.float32, 1)
            if ids is None or positions is None or position_frequencies.shape[0] < (width + 1) // 2:
                raise KernelError("stream_norm: a position vector needs ids, positions and a frequency for every two columns")
            self._check(positions, "positions", torch.int32, 1)
        count = stream.shape[0]
        if rows is not None:
            self._check(rows, "rows", torch.int32, 1)
            count = rows.shape[0]
        out = None
        if w_open is not None:
            out = torch.empty((count, width), dtype=dtype, device=stream.device)
        self._call("ts_stream_norm", _ptr(branch), _ptr(w_close), _ptr(stream), _ptr(w_open), _ptr(out), _ptr(rows), count,
                   width, eps, _ptr(table), _ptr(ids), table.shape[0] if table is not None else 0, scale,
                   (1 if centered else 0) | (2 if plain_add else 0), _DTYPE_CODE[dtype],
                   _ptr(positions) if position_frequencies is not None else 0, _ptr(position_frequencies), _ptr(w_start),
                   _stream())
        return out

    # ------------------------------------------------------------------ linear recurrences
    def linear_recurrence(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ctx, binding, *, heads: int, dim: int,
                          vdim: int, z: torch.Tensor | None, bias: torch.Tensor | None, head_decays: torch.Tensor | None,
                          inv_tau: float, q_scale: float, k_scale: float, position=None) -> torch.Tensor:
        """
        float32 [T, heads * vdim]: o_t = S_t^T q_t with S_t = diag(a_t) S_(t-1) + k_t v_t^T per request and
        head, the state read from and written back to the request's slot (`binding.state`).  q, k, v are
        column slices of one projection output (unit stride inside a row).  Decays: `z` (float32
        [T, heads * dim] logits, a = sigmoid(z + bias)^inv_tau) or `head_decays` (float32 [heads]).
        """
        for t, name, cols in ((q, "q", heads * dim), (k, "k", heads * dim), (v, "v", heads * vdim)):
            if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.shape[1] != cols or t.dtype not in _DTYPE_CODE:
                raise KernelError(f"linear_recurrence: {name} must be a CUDA [T, {cols}] slice with unit column stride")
        if binding is None or binding.state is None or binding.state_slots is None:
            raise KernelError("linear_recurrence: the cache entry has no state slot")
        state = binding.state
        if state.stride(1) != 1 or state.stride(0) % 4 or state.data_ptr() % 4 or state.shape[1] < heads * dim * vdim * 4:
            raise KernelError("linear_recurrence: the state rows are not float32-aligned or too small")
        T = q.shape[0]
        if z is not None:
            self._check(z, "decay logits", torch.float32, 2)
            if tuple(z.shape) != (T, heads * dim):
                raise KernelError(f"linear_recurrence: decay logits are {tuple(z.shape)}, expected {(T, heads * dim)}")
        freq, rot = None, 0
        if position is not None:
            freq, rot = position.frequencies, position.dims
        out = torch.empty((T, heads * vdim), dtype=torch.float32, device=q.device)
        prepared = torch.empty((3, T, heads * dim), dtype=torch.float32, device=q.device)   # q, k, decays as they enter the scan
        self._call("ts_linear_recurrence", _ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), _ptr(z),
                   z.stride(0) if z is not None else 0, _ptr(bias), _ptr(head_decays), inv_tau, q_scale, k_scale,
                   _ptr(freq), rot, _ptr(ctx.positions), _ptr(ctx.cu_q), _ptr(binding.state_slots),
                   binding.state_slots.shape[0], state.data_ptr(), state.stride(0) // 4, _ptr(out), heads, dim, vdim,
                   T, _ptr(prepared), _DTYPE_CODE[q.dtype], _stream())
        self.launches += 1                                   # the kernel that prepares the scan's inputs
        return out

    def head_norm_gate(self, o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor | None, heads: int, vdim: int,
                       eps: float, dtype: torch.dtype, *, gate_kind: str = "silu", weight_per_head: bool = False,
                       log_max: torch.Tensor | None = None, scale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
        """
        [T, heads * vdim] in `dtype`: each head's o (float32) RMS-normed over vdim, times weight (if any; one
        stretch of vdim shared by the heads, or heads * vdim with `weight_per_head`), times silu or sigmoid of
        the gate, times `scale`.  With `log_max` (float32 [T, heads]) o holds vdim + 1 columns a head and is
        first divided by max(|o[.., vdim]|, exp(-log_max)) + 1e-6.  `out` may be a column stretch of a wider tensor.
        """
        self._check(o, "o", torch.float32, 2)
        T = o.shape[0]
        o_head = vdim + 1 if log_max is not None else vdim
        if o.shape[1] != heads * o_head:
            raise KernelError(f"head_norm_gate: o has {o.shape[1]} columns, expected {heads * o_head}")
        if gate.stride(1) != 1 or gate.dtype != dtype or tuple(gate.shape) != (T, heads * vdim):
            raise KernelError("head_norm_gate: the gate must be a [T, heads * vdim] slice of the activation dtype")
        if weight is not None and weight.numel() != (heads * vdim if weight_per_head else vdim):
            raise KernelError(f"head_norm_gate: the weight has {weight.numel()} elements")
        if gate_kind not in ("silu", "sigmoid"):
            raise KernelError(f"head_norm_gate: gate kind {gate_kind!r}")
        if out is None:
            out = torch.empty((T, heads * vdim), dtype=dtype, device=o.device)
        elif out.dtype != dtype or tuple(out.shape) != (T, heads * vdim) or out.stride(1) != 1:
            raise KernelError("head_norm_gate: out must be a [T, heads * vdim] stretch of the activation dtype")
        self._call("ts_head_norm_gate", _ptr(o), o_head, _ptr(gate), gate.stride(0), _ptr(weight),
                   vdim if weight_per_head else 0, _ptr(log_max), _ptr(out), out.stride(0), T, heads, vdim, eps,
                   1 if gate_kind == "sigmoid" else 0, scale, _DTYPE_CODE[dtype], _stream())
        return out

    # ------------------------------------------------------------------ attention with normed queries and keys, gated recurrences
    def qk_norm_rope_store(self, y: torch.Tensor, offsets: tuple[int, int, int], biases, weights, eps: float, position,
                           ctx, binding, heads: int, kv_heads: int, dim: int, vdim: int, *, norm_per_head: bool = False,
                           q_temperature: tuple[float, int] | None = None, value_heads: int = 0) -> torch.Tensor:
        """
        From the projection's output y (q, k, v at the column `offsets`): biases added (float32 tensors or
        None), q and k RMS-normed over the whole projection with `weights` (q's, k's; or None; with
        `norm_per_head` every head by itself, the weights [dim]), rotated by `position` (frequencies, dims,
        magnitude), q multiplied by 1 + coef * ln(floor((position + 1) / every) + 1) for `q_temperature`
        (coef, every), k and v stored into the token's cache slot.  `value_heads` (0: as many as key heads): v
        holds that many heads of vdim channels.  Returns q [T, heads * dim].
        """
        if y.dtype not in _DTYPE_CODE or y.dim() != 2 or y.stride(1) != 1:
            raise KernelError("qk_norm_rope_store: y must be a [T, columns] stretch of an activation dtype")
        if binding.k_pool.dtype != y.dtype:
            raise KernelError(f"cache pool is {binding.k_pool.dtype} but activations are {y.dtype}")
        T = y.shape[0]
        q = torch.empty((T, heads * dim), dtype=y.dtype, device=y.device)
        freq, rot, magnitude = None, 0, 1.0
        if position is not None:
            freq, rot, magnitude = position.frequencies, position.dims, float(getattr(position, "magnitude", 1.0))
        qb, kb, vb = biases if biases is not None else (None, None, None)
        qw, kw = weights if weights is not None else (None, None)
        for w in (qw, kw):
            if w is not None and w.numel() != (dim if norm_per_head else (heads if w is qw else kv_heads) * dim):
                raise KernelError(f"qk_norm_rope_store: a norm weight of {w.numel()} elements")
        coef, every = q_temperature if q_temperature is not None else (0.0, 0)
        v_page_stride, v_entry_offset = binding.value_geometry()
        self._call("ts_qk_norm_rope_store", _ptr(y), y.stride(0), offsets[0], offsets[1], offsets[2], _ptr(qb), _ptr(kb),
                   _ptr(vb), _ptr(qw), _ptr(kw), eps, _ptr(freq), rot, magnitude, _ptr(ctx.positions),
                   _ptr(ctx.seq_of_token), _ptr(q), _ptr(binding.k_pool), _ptr(binding.v_pool), binding.page_stride,
                   binding.entry_offset, v_page_stride, v_entry_offset, binding.page_tokens, binding.num_pages,
                   _ptr(binding.block_table), binding.table_width, 1 if binding.writes else 0, T, heads, kv_heads, dim,
                   vdim, _DTYPE_CODE[y.dtype], 1 if norm_per_head else 0, float(coef), int(every), int(value_heads), _stream())
        return q

    def paged_attention_split(self, q: torch.Tensor, ctx, binding, nh: int, nkv: int, hd: int, vd: int, scale: float,
                              window: int, *, weights: str = "softmax", slopes: torch.Tensor | None = None,
                              head_bias: torch.Tensor | None = None, head_gate: torch.Tensor | None = None,
                              softcap: float = 0.0, chunk: int = 0, value_heads: int = 0,
                              out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """
        [T, nh * vd]: causal attention of q [T, nh * hd] over the entry's cached keys (head size hd) and
        values (head size vd).  Equal head sizes of 64 or 128 in bfloat16 run on the tensor-core kernels
        (`paged_attention`), everything else on the generic kernel.

        Options: `slopes` (float32 [nh]) takes slopes[h] * (i - j) off the score of query i and key j,
        `head_bias` (float32 [nh]) is added to every score of its head, `weights` "sigmoid" makes a visible
        key's weight sigmoid(score) with no normalisation, `head_gate` ([T, nh] logits, a column stretch of
        the activation dtype) multiplies head h's output by sigmoid(head_gate[t, h]); `softcap` c > 0 turns the
        scaled product into c tanh(. / c); `chunk` n > 0 hides every key before floor(i / n) * n from query i;
        `value_heads` g > 0: the value pool holds g heads and head h reads value head h / (nh / g); `out_dtype`
        float32 keeps the output unrounded.
        """
        self._check(q, "q", tuple(_DTYPE_CODE), 2)
        if q.shape[1] != nh * hd:
            raise KernelError(f"paged_attention_split: q has {q.shape[1]} columns, expected {nh * hd}")
        if weights not in ("softmax", "sigmoid"):
            raise KernelError(f"paged_attention_split: weights {weights!r}")
        if softcap < 0 or chunk < 0 or value_heads < 0 or (value_heads and (nkv % value_heads or nh % value_heads)):
            raise KernelError(f"paged_attention_split: softcap {softcap}, chunk {chunk}, {value_heads} value heads for {nkv} key heads")
        if out_dtype not in (None, q.dtype, torch.float32):
            raise KernelError(f"paged_attention_split: output dtype {out_dtype}")
        out_f32 = out_dtype == torch.float32 and q.dtype != torch.float32
        if (weights != "softmax" or slopes is not None or head_bias is not None or head_gate is not None or softcap > 0
                or chunk > 0 or value_heads > 0 or out_f32):
            return self._paged_attention_scored(q, ctx, binding, nh, nkv, hd, vd, scale, window, weights, slopes, head_bias,
                                                head_gate, softcap, chunk, value_heads, out_f32)
        if (hd == vd and q.dtype == torch.bfloat16 and getattr(ctx, "cu_q", None) is not None
                and self.lib.ts_attention_bf16_supported(hd, binding.page_tokens, nh, nkv)):
            # the tensor-core kernels read q from the columns of a [q | k | v] row: q alone is such a row's first part
            qkv = torch.empty((q.shape[0], (nh + 2 * nkv) * hd), dtype=q.dtype, device=q.device)
            qkv[:, :nh * hd].copy_(q)
            return self.paged_attention(qkv, ctx, binding, nh, nkv, hd, scale, window)
        out = torch.empty((q.shape[0], nh * vd), dtype=q.dtype, device=q.device)
        v_page_stride, v_entry_offset = binding.value_geometry()
        self._call("ts_paged_attention_split", _ptr(q), q.stride(0), _ptr(out), _ptr(binding.k_pool), _ptr(binding.v_pool),
                   binding.page_stride, binding.entry_offset, v_page_stride, v_entry_offset, binding.page_tokens,
                   binding.num_pages, _ptr(binding.block_table), binding.table_width, _ptr(ctx.positions),
                   _ptr(ctx.seq_of_token), q.shape[0], nh, nkv, hd, vd, scale, window, _DTYPE_CODE[q.dtype], _stream())
        return out

    def _paged_attention_scored(self, q, ctx, binding, nh, nkv, hd, vd, scale, window, weights, slopes, head_bias,
                                head_gate, softcap=0.0, chunk=0, value_heads=0, out_f32=False) -> torch.Tensor:
        for t, name in ((slopes, "slopes"), (head_bias, "head bias")):
            if t is not None:
                self._check(t, name, torch.float32, 1)
                if t.shape[0] != nh:
                    raise KernelError(f"paged_attention_split: {name} has {t.shape[0]} elements for {nh} heads")
        if head_gate is not None and (head_gate.dtype != q.dtype or head_gate.dim() != 2 or head_gate.stride(1) != 1
                                      or tuple(head_gate.shape) != (q.shape[0], nh)):
            raise KernelError("paged_attention_split: the head gate must be a [T, heads] stretch of the activation dtype")
        out = torch.empty((q.shape[0], nh * vd), dtype=torch.float32 if out_f32 else q.dtype, device=q.device)
        plain = softcap == 0 and chunk == 0 and value_heads == 0 and not out_f32
        if (weights == "softmax" and slopes is None and head_bias is None and head_gate is None and not out_f32
                and self.tensor_core_attention(q, binding, nh, nkv, hd, vd, ctx)):
            # the tensor-core kernels with the mask's and the score's options: tiles of a prompt's portion, split keys
            # for requests that feed one token
            num_seqs = ctx.ctx_lens.shape[0]
            prefill_seqs = getattr(ctx, "prefill_seqs", None)
            num_prefill = prefill_seqs.shape[0] if prefill_seqs is not None else 0
            decode_ctx = getattr(ctx, "max_decode_ctx_len", ctx.max_ctx_len)
            scratch, floats = None, 0
            if ctx.min_q_len <= 1:
                floats = self.lib.ts_attention_bf16_scratch_floats(num_seqs, nh, hd, decode_ctx)
                key = ("attention", floats)
                scratch = ctx.scratch.get(key)
                if scratch is None:
                    scratch = ctx.scratch[key] = torch.empty((floats,), dtype=torch.float32, device=q.device)
            max_q_len = ctx.max_q_len
            if (max_q_len > 1 and self.tcgen05_attention and self.lib.ts_attention_tcgen05_supported(
                    hd, binding.page_tokens, nh, nkv, 0)):
                # prompt portions on the tcgen05 kernel; requests that feed one token stay with the split-key kernels
                per_entry = nkv * binding.page_tokens * hd
                self._call("ts_prefill_attention_tcgen05_masked", _ptr(q), q.stride(0), _ptr(out), _ptr(binding.k_pool),
                           _ptr(binding.v_pool), binding.num_pages, binding.page_stride // per_entry,
                           binding.entry_offset // per_entry, binding.page_tokens, _ptr(binding.block_table),
                           binding.table_width, _ptr(ctx.cu_q), _ptr(ctx.ctx_lens), num_seqs, q.shape[0], max_q_len, nh, nkv,
                           hd, scale, window, int(chunk), float(softcap), int(value_heads), _ptr(prefill_seqs), num_prefill,
                           self.error_word().data_ptr(), _stream())
                if ctx.min_q_len > 1:
                    return out
                max_q_len = 1
            v_page_stride, v_entry_offset = binding.value_geometry()
            self._call("ts_paged_attention_bf16_masked", _ptr(q), q.stride(0), _ptr(out), _ptr(binding.k_pool),
                       _ptr(binding.v_pool), binding.page_stride, binding.entry_offset, v_page_stride, v_entry_offset,
                       binding.page_tokens, binding.num_pages, _ptr(binding.block_table), binding.table_width, _ptr(ctx.cu_q),
                       _ptr(ctx.ctx_lens), num_seqs, max_q_len, min(ctx.min_q_len, max_q_len), decode_ctx, nh, nkv, hd, scale, window,
                       int(chunk), float(softcap), int(value_heads), _ptr(scratch), floats, _ptr(prefill_seqs), num_prefill,
                       _stream())
            if ctx.min_q_len <= 1:
                self.launches += 1 if max_q_len <= 1 else 2          # decode + combine (+ prefill) in one call
            return out
        if (plain and weights == "sigmoid" and hd == vd and q.dtype == torch.bfloat16 and getattr(ctx, "cu_q", None) is not None
                and q.stride(0) % 8 == 0 and self.lib.ts_attention_bf16_supported(hd, binding.page_tokens, nh, nkv)):
            # the tensor-core kernels: tiles of a prompt's portion, split keys for requests that feed one token
            num_seqs = ctx.ctx_lens.shape[0]
            prefill_seqs = getattr(ctx, "prefill_seqs", None)
            num_prefill = prefill_seqs.shape[0] if prefill_seqs is not None else 0
            decode_ctx = getattr(ctx, "max_decode_ctx_len", ctx.max_ctx_len)
            scratch, floats = None, 0
            max_q_len = ctx.max_q_len
            gate_stride = head_gate.stride(0) if head_gate is not None else 0
            if (max_q_len > 1 and self.tcgen05_attention and self.lib.ts_attention_tcgen05_supported(
                    hd, binding.page_tokens, nh, nkv, 0)):
                # prompt portions on the tcgen05 kernel; requests that feed one token stay with the split-key kernels
                per_entry = nkv * binding.page_tokens * hd
                self._call("ts_prefill_attention_tcgen05_sigmoid", _ptr(q), q.stride(0), _ptr(out), _ptr(binding.k_pool),
                           _ptr(binding.v_pool), binding.num_pages, binding.page_stride // per_entry,
                           binding.entry_offset // per_entry, binding.page_tokens, _ptr(binding.block_table),
                           binding.table_width, _ptr(ctx.cu_q), _ptr(ctx.ctx_lens), num_seqs, q.shape[0], max_q_len, nh, nkv,
                           hd, scale, window, _ptr(slopes), _ptr(head_bias), _ptr(head_gate), gate_stride,
                           _ptr(prefill_seqs), num_prefill, self.error_word().data_ptr(), _stream())
                if ctx.min_q_len > 1:
                    return out
                max_q_len = 1
            if ctx.min_q_len <= 1:
                floats = self.lib.ts_attention_bf16_scratch_floats(num_seqs, nh, hd, decode_ctx)
                key = ("attention", floats)
                scratch = ctx.scratch.get(key)
                if scratch is None:
                    scratch = ctx.scratch[key] = torch.empty((floats,), dtype=torch.float32, device=q.device)
            self._call("ts_paged_attention_bf16_sigmoid", _ptr(q), q.stride(0), _ptr(out), _ptr(binding.k_pool),
                       _ptr(binding.v_pool), binding.page_stride, binding.entry_offset, binding.page_tokens,
                       binding.num_pages, _ptr(binding.block_table), binding.table_width, _ptr(ctx.cu_q),
                       _ptr(ctx.ctx_lens), num_seqs, max_q_len, min(ctx.min_q_len, max_q_len), decode_ctx, nh, nkv, hd,
                       scale, window, _ptr(scratch), floats, _ptr(prefill_seqs), num_prefill, _ptr(slopes),
                       _ptr(head_bias), _ptr(head_gate), gate_stride, _stream())
            if ctx.min_q_len <= 1:
                self.launches += 1 if max_q_len <= 1 else 2          # decode + combine (+ prefill) in one call
            return out
        v_page_stride, v_entry_offset = binding.value_geometry()
        self._call("ts_paged_attention_scored", _ptr(q), q.stride(0), _ptr(out), _ptr(binding.k_pool), _ptr(binding.v_pool),
                   binding.page_stride, binding.entry_offset, v_page_stride, v_entry_offset, binding.page_tokens,
                   binding.num_pages, _ptr(binding.block_table), binding.table_width, _ptr(ctx.positions),
                   _ptr(ctx.seq_of_token), q.shape[0], nh, nkv, hd, vd, scale, window, _DTYPE_CODE[q.dtype],
                   1 if weights == "sigmoid" else 0, _ptr(slopes), _ptr(head_bias), _ptr(head_gate),
                   head_gate.stride(0) if head_gate is not None else 0, float(softcap), int(chunk), int(value_heads),
                   1 if out_f32 else 0, _stream())
        return out

    def dense_prompt_attention_supported(self, q: torch.Tensor, nh: int, nkv: int, hd: int) -> bool:
        """Whether `dense_prompt_attention` takes these sizes (bfloat16, heads of 64 or 128 channels, aligned query rows)."""
        return bool(q.dtype == torch.bfloat16 and q.dim() == 2 and q.stride(1) == 1 and q.stride(0) % 8 == 0
                    and q.data_ptr() % 16 == 0 and self.tcgen05_attention
                    and self.lib.ts_attention_tcgen05_supported(hd, 64, nh, nkv, 0))

    def dense_prompt_attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kv_start: torch.Tensor, ctx, nh: int,
                               nkv: int, hd: int, scale: float, out: torch.Tensor | None = None) -> torch.Tensor:
        """
        Causal softmax attention of the step's prompt portions (requests that feed more than one token) over keys
        and values worked out for the step: k, v [rows, nkv * hd] bfloat16, request s's key j in row kv_start[s] + j
        (int32 [requests] on the device), ctx.ctx_lens[s] keys a request.  Rows of requests that feed one token are
        left as they are in `out` ([T, nh * hd]; made here if not given).  The tcgen05 prompt kernel.
        """
        self._check_rows(q, "q")
        self._check(k, "k", torch.bfloat16, 2)
        self._check(v, "v", torch.bfloat16, 2)
        self._check(kv_start, "kv_start", torch.int32, 1)
        if k.shape != v.shape or k.shape[1] != nkv * hd or q.shape[1] != nh * hd or kv_start.shape[0] != ctx.ctx_lens.shape[0]:
            raise KernelError(f"dense_prompt_attention: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)} for "
                              f"{nh}:{nkv} heads of {hd}")
        if not self.dense_prompt_attention_supported(q, nh, nkv, hd):
            raise KernelError(f"dense_prompt_attention: sizes not taken ({nh}:{nkv} heads of {hd}, {q.dtype})")
        if out is None:
            out = torch.empty((q.shape[0], nh * hd), dtype=q.dtype, device=q.device)
        prefill_seqs = getattr(ctx, "prefill_seqs", None)
        num_prefill = prefill_seqs.shape[0] if prefill_seqs is not None else 0
        self._call("ts_prefill_attention_tcgen05_dense", _ptr(q), q.stride(0), _ptr(out), _ptr(k), _ptr(v), k.shape[0],
                   _ptr(kv_start), _ptr(ctx.cu_q), _ptr(ctx.ctx_lens), ctx.ctx_lens.shape[0], q.shape[0], ctx.max_q_len, nh, nkv,
                   hd, scale, _ptr(prefill_seqs), num_prefill, self.error_word().data_ptr(), _stream())
        return out

    def tensor_core_attention(self, q: torch.Tensor, binding, nh: int, nkv: int, hd: int, vd: int, ctx=None) -> bool:
        """Whether the bfloat16 tensor-core attention kernels take these sizes (else the generic kernel runs)."""
        return bool(hd == vd and q.dtype == torch.bfloat16 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
                    and (ctx is None or getattr(ctx, "cu_q", None) is not None)
                    and self.lib.ts_attention_bf16_supported(hd, binding.page_tokens, nh, nkv))

    def difference_head_norm(self, maps: torch.Tensor, ctx, heads: int, kv_heads: int, vdim: int, weight: float, eps: float,
                             out_scale: float, dtype: torch.dtype) -> torch.Tensor:
        """
        Differential attention's last step.  maps [T, 2 * heads * vdim] (float32 or `dtype`) holds per token the two
        maps' outputs in the order [key/value group][map][head in group][vdim]; returns [T, heads * vdim] in `dtype`:
        per head (a_1 - weight * a_2) / sqrt(mean(.^2) + eps) * out_scale, heads in their own order.
        """
        self._check(maps, "maps", (torch.float32, dtype), 2)
        if maps.shape[1] != 2 * heads * vdim or heads % kv_heads:
            raise KernelError(f"difference_head_norm: rows of {maps.shape[1]} for {heads} heads of {vdim} over {kv_heads} groups")
        out = torch.empty((maps.shape[0], heads * vdim), dtype=dtype, device=maps.device)
        self._call("ts_difference_head_norm", _ptr(maps), maps.stride(0), 1 if maps.dtype == torch.float32 else 0, _ptr(out),
                   out.stride(0), _ptr(ctx.seq_of_token), maps.shape[0], heads, kv_heads, vdim, float(weight), float(eps),
                   float(out_scale), _DTYPE_CODE[dtype], _stream())
        return out

    def scale_tanh_cap(self, x: torch.Tensor, scale: float, cap: float) -> torch.Tensor:
        """x (float32, in place) <- cap * tanh(x * scale / cap), or x * scale where cap is 0."""
        self._check(x, "x", torch.float32)
        self._call("ts_scale_tanh_cap", _ptr(x), x.numel(), float(scale), float(cap), _stream())
        return x

    def mingru_scan(self, y: torch.Tensor, offsets: tuple[int, int, int], z_bias: torch.Tensor | None,
                    x_bias: torch.Tensor | None, ctx, binding, width: int, dtype: torch.dtype) -> torch.Tensor:
        """
        [T, width] in `dtype`: S_t * silu(g_t) of the element-wise gated recurrence S_t = (1 - z_t) S_(t-1) + z_t c_t
        with z = sigmoid(a + z_bias), c = u + x_bias + 1/2 where u + x_bias >= 0 and sigmoid(u + x_bias) below.
        a, u, g are the stretches of `width` columns of y (float32 or `dtype`) at the column `offsets`; the
        state (float32 [width]) is read from and written back to the request's slot.
        """
        if y.dim() != 2 or y.stride(1) != 1 or y.dtype not in (torch.float32, dtype) or dtype not in _DTYPE_CODE:
            raise KernelError("mingru_scan: y must be a [T, columns] stretch, float32 or of the activation dtype")
        if max(offsets) + width > y.shape[1]:
            raise KernelError(f"mingru_scan: y has {y.shape[1]} columns, fewer than the stretches at {offsets} need")
        for b, name in ((z_bias, "z bias"), (x_bias, "x bias")):
            if b is not None:
                self._check(b, name, torch.float32, 1)
                if b.shape[0] != width:
                    raise KernelError(f"mingru_scan: the {name} has {b.shape[0]} elements for {width} channels")
        state, stride = self._state_floats(binding, width, "mingru_scan")
        T = y.shape[0]
        out = torch.empty((T, width), dtype=dtype, device=y.device)
        self._call("ts_mingru_scan", _ptr(y), y.stride(0), offsets[0], offsets[1], offsets[2], _DTYPE_CODE[y.dtype],
                   _ptr(z_bias), _ptr(x_bias), _ptr(ctx.cu_q), _ptr(binding.state_slots), binding.state_slots.shape[0],
                   state.data_ptr(), stride, _ptr(out), width, T, int(getattr(ctx, "max_q_len", 0) or 0),
                   _DTYPE_CODE[dtype], _stream())
        return out

    UNARY_ACTIVATIONS = {"relu2": 0, "xielu": 1}

    def unary_activation(self, x: torch.Tensor, kind: str, a: float = 0.0, b: float = 0.0) -> torch.Tensor:
        """act(x), in place: "relu2" relu(x)^2; "xielu" a x^2 + x/2 for x > 0 and b (exp(x) - 1 - x) + x/2 for x <= 0."""
        self._check(x, "x", tuple(_DTYPE_CODE))
        if kind not in self.UNARY_ACTIVATIONS:
            raise KernelError(f"unary_activation: kind {kind!r} of {sorted(self.UNARY_ACTIVATIONS)}")
        self._call("ts_unary_activation_rows", _ptr(x), _ptr(x), x.numel(), self.UNARY_ACTIVATIONS[kind], float(a), float(b),
                   _DTYPE_CODE[x.dtype], _stream())
        return x

    def sigmoid_gate(self, a: torch.Tensor, gate: torch.Tensor, scale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
        """a * sigmoid(gate) * scale, [T, cols]; the operands and `out` may be column stretches of wider tensors."""
        if a.dtype not in _DTYPE_CODE or gate.dtype != a.dtype or a.shape != gate.shape or a.stride(1) != 1 or gate.stride(1) != 1:
            raise KernelError("sigmoid_gate: a and gate must be [T, cols] stretches of one activation dtype")
        if out is None:
            out = torch.empty(a.shape, dtype=a.dtype, device=a.device)
        elif out.dtype != a.dtype or out.shape != a.shape or out.stride(1) != 1:
            raise KernelError("sigmoid_gate: out must be a [T, cols] stretch of the activation dtype")
        self._call("ts_sigmoid_gate", _ptr(a), a.stride(0), _ptr(gate), gate.stride(0), _ptr(out), out.stride(0), a.shape[0],
                   a.shape[1], scale, _DTYPE_CODE[a.dtype], _stream())
        return out

    @staticmethod
    def _state_floats(binding, floats: int, what: str) -> tuple[torch.Tensor, int]:
        if binding is None or binding.state is None or binding.state_slots is None:
            raise KernelError(f"{what}: the cache entry has no state slot")
        state = binding.state
        if state.stride(1) != 1 or state.stride(0) % 4 or state.data_ptr() % 4 or state.shape[1] < floats * 4:
            raise KernelError(f"{what}: the state rows are not float32-aligned or too small")
        return state, state.stride(0) // 4

    def short_conv_silu(self, x: torch.Tensor, taps: torch.Tensor, ctx, binding) -> torch.Tensor:
        """
        float32 [T, C]: silu of the causal convolution over time of x [T, C] (a column stretch) with
        taps [C, K] (float32, the last column is the current token's); the K - 1 inputs before this step's
        first token come from the request's state slot ([K - 1, C] float32), which is moved on.
        """
        if x.dtype not in _DTYPE_CODE or x.dim() != 2 or x.stride(1) != 1:
            raise KernelError("short_conv_silu: x must be a [T, C] stretch of an activation dtype")
        self._check(taps, "taps", torch.float32, 2)
        T, C = x.shape
        K = taps.shape[1]
        if taps.shape[0] != C:
            raise KernelError(f"short_conv_silu: {taps.shape[0]} filters for {C} channels")
        state, stride = self._state_floats(binding, (K - 1) * C, "short_conv_silu")
        y = torch.empty((T, C), dtype=torch.float32, device=x.device)
        self._call("ts_short_conv_silu", _ptr(x), x.stride(0), _ptr(taps), _ptr(ctx.seq_of_token), _ptr(ctx.cu_q),
                   _ptr(binding.state_slots), binding.state_slots.shape[0], state.data_ptr(), stride, _ptr(y), T, C, K,
                   _DTYPE_CODE[x.dtype], _stream())
        if K > 1:
            self.launches += 1                               # the kernel that moves the slot on
        return y

    def recurrence_scan(self, prepared: torch.Tensor, v: torch.Tensor, ctx, binding, *, heads: int, dim: int, vdim: int,
                        v_cols: int | None = None, beta: torch.Tensor | None = None) -> torch.Tensor:
        """
        float32 [T, heads * vdim]: the scan of `linear_recurrence` from inputs the caller prepared: prepared
        float32 [3, T, heads * dim] (q, k, decay), v [T, heads * v_cols] (float32 or an activation dtype; value
        columns from v_cols to vdim are the constant 1), `beta` float32 [T, heads] for the delta rule.
        The state slot holds [heads, dim, vdim] floats.
        """
        T = prepared.shape[1]
        v_cols = vdim if v_cols is None else v_cols
        self._check(prepared, "prepared", torch.float32, 3)
        if tuple(prepared.shape) != (3, T, heads * dim):
            raise KernelError(f"recurrence_scan: prepared is {tuple(prepared.shape)}, expected {(3, T, heads * dim)}")
        if v.dtype not in _DTYPE_CODE or v.dim() != 2 or v.stride(1) != 1 or tuple(v.shape) != (T, heads * v_cols):
            raise KernelError(f"recurrence_scan: v must be a [T, {heads * v_cols}] stretch")
        if beta is not None:
            self._check(beta, "beta", torch.float32, 2)
            if tuple(beta.shape) != (T, heads):
                raise KernelError(f"recurrence_scan: beta is {tuple(beta.shape)}, expected {(T, heads)}")
        state, stride = self._state_floats(binding, heads * dim * vdim, "recurrence_scan")
        out = torch.empty((T, heads * vdim), dtype=torch.float32, device=v.device)
        self._call("ts_recurrence_scan", _ptr(prepared), _ptr(v), v.stride(0), v_cols, _DTYPE_CODE[v.dtype], _ptr(beta),
                   _ptr(ctx.cu_q), _ptr(binding.state_slots), binding.state_slots.shape[0], state.data_ptr(), stride,
                   _ptr(out), heads, dim, vdim, T, _stream())
        return out

    def delta_prepare(self, q: torch.Tensor, k: torch.Tensor, z: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
                      b: torch.Tensor, *, heads: int, kv_heads: int, dim: int, unit_eps: float, q_scale: float):
        """
        (prepared [3, T, heads * dim], beta [T, heads]), float32, for the delta rule's scan: q, k (float32
        [T, kv_heads * dim] stretches with one row stride) as unit vectors per head, q scaled; decays
        exp(-exp(a_log) softplus(z + dt_bias)); beta = sigmoid(b).
        """
        T = q.shape[0]
        for t, name, cols in ((q, "q", kv_heads * dim), (k, "k", kv_heads * dim)):
            if t.dtype != torch.float32 or t.stride(1) != 1 or tuple(t.shape) != (T, cols):
                raise KernelError(f"delta_prepare: {name} must be a float32 [T, {cols}] stretch")
        if q.stride(0) != k.stride(0):
            raise KernelError("delta_prepare: q and k must share a row stride")
        self._check(z, "decay logits", torch.float32, 2)
        if tuple(z.shape) != (T, heads * dim) or b.dtype not in _DTYPE_CODE or b.stride(1) != 1 or tuple(b.shape) != (T, heads):
            raise KernelError("delta_prepare: decay logits [T, heads * dim] and beta logits [T, heads] are needed")
        prepared = torch.empty((3, T, heads * dim), dtype=torch.float32, device=q.device)
        beta = torch.empty((T, heads), dtype=torch.float32, device=q.device)
        self._call("ts_delta_prepare", _ptr(q), _ptr(k), q.stride(0), _ptr(z), _ptr(dt_bias), _ptr(a_log), _ptr(b),
                   b.stride(0), _ptr(prepared), _ptr(beta), T, heads, kv_heads, dim, unit_eps, q_scale,
                   _DTYPE_CODE[b.dtype], _stream())
        return prepared, beta

    def mlstm_prepare(self, q: torch.Tensor, k: torch.Tensor, gates: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor,
                      ctx, binding, *, heads: int, dim: int, cap: float, q_scale: float, max_offset_floats: int):
        """
        (prepared [3, T, heads * dim], log_max [T, heads]) for the scan of a matrix memory with exponential
        gates.  q, k: [T, heads * dim] stretches of one activation dtype; gates: float32 [T, 2 heads],
        input gates then forget gates, before bias and cap.  The running maxima ([heads] floats) live
        `max_offset_floats` floats into the request's state slot.
        """
        T = q.shape[0]
        for t, name in ((q, "q"), (k, "k")):
            if t.dtype not in _DTYPE_CODE or t.stride(1) != 1 or tuple(t.shape) != (T, heads * dim) or t.dtype != q.dtype:
                raise KernelError(f"mlstm_prepare: {name} must be a [T, {heads * dim}] stretch of the activation dtype")
        if gates.dtype != torch.float32 or gates.stride(1) != 1 or tuple(gates.shape) != (T, 2 * heads):
            raise KernelError("mlstm_prepare: the gates must be float32 [T, 2 heads]")
        state, stride = self._state_floats(binding, max_offset_floats + heads, "mlstm_prepare")
        dev = q.device
        prepared = torch.empty((3, T, heads * dim), dtype=torch.float32, device=dev)
        log_max = torch.empty((T, heads), dtype=torch.float32, device=dev)
        factors = torch.empty((2, T, heads), dtype=torch.float32, device=dev)
        self._call("ts_mlstm_prepare", _ptr(q), _ptr(k), q.stride(0), k.stride(0), _ptr(gates),
                   gates.data_ptr() + heads * gates.element_size(), gates.stride(0), _ptr(bias_i), _ptr(bias_f), cap, q_scale,
                   _ptr(ctx.cu_q), _ptr(binding.state_slots), binding.state_slots.shape[0],
                   state.data_ptr() + 4 * max_offset_floats, stride, _ptr(log_max), _ptr(factors), _ptr(prepared), T, heads,
                   dim, _DTYPE_CODE[q.dtype], _stream())
        self.launches += 1                                   # gates, then what enters the scan
        return prepared, log_max

    # ------------------------------------------------------------------ attention over a cached latent
    def latent_prepare(self, y: torch.Tensor, ctx, binding, q_rank: int, rank: int, rot: int, q_weight: torch.Tensor,
                       kv_weight: torch.Tensor, eps: float, freq: torch.Tensor) -> torch.Tensor:
        """
        y [T, q_rank + rank + rot] (the down projections' output, or a column stretch of it): returns the normed
        query latent [T, q_rank] and stores [norm(c) | rotated k_rot] into each token's slot of the cache entry.
        q_rank 0 (queries without a latent) and rot 0 (no rotated part, `freq` None) are allowed.
        """
        if y.dtype not in _DTYPE_CODE or y.dim() != 2 or y.stride(1) != 1 or not y.is_cuda:
            raise KernelError("latent_prepare: y must be a [T, columns] stretch of an activation dtype on the device")
        if y.shape[1] != q_rank + rank + rot:
            raise KernelError(f"latent_prepare: rows of {y.shape[1]} columns, expected {q_rank + rank + rot}")
        if binding.k_pool.dtype != y.dtype:
            raise KernelError(f"cache pool is {binding.k_pool.dtype} but activations are {y.dtype}")
        c_q = torch.empty((y.shape[0], q_rank), dtype=y.dtype, device=y.device)
        self._call("ts_latent_prepare", _ptr(y), y.stride(0), q_rank, rank, rot, _ptr(q_weight), _ptr(kv_weight), eps,
                   _ptr(freq), _ptr(ctx.positions), _ptr(ctx.seq_of_token), _ptr(c_q), _ptr(binding.k_pool),
                   binding.page_stride, binding.entry_offset, binding.page_tokens, binding.num_pages,
                   _ptr(binding.block_table), binding.table_width, 1 if binding.writes else 0, y.shape[0],
                   _DTYPE_CODE[y.dtype], _stream())
        return c_q

    def per_head_linear(self, x: torch.Tensor, w: torch.Tensor, heads: int, head_width: int, k: int,
                        out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """
        [T, heads, N]: head h's first k channels of x [T, heads * head_width] times w[h]^T, w [heads, N, k].
        float32: the engine's FFMA kernel, one product per head in one launch; bfloat16: the library's
        batched product.  x may be a column stretch of wider rows; the result may be a strided view.
        """
        self._check_rows(x, "x")
        self._check(w, "w", x.dtype, 3)
        T, N = x.shape[0], w.shape[1]
        if x.shape[1] != heads * head_width or w.shape[0] != heads or w.shape[2] != k or k > head_width:
            raise KernelError(f"per_head_linear: x {tuple(x.shape)}, w {tuple(w.shape)} do not fit {heads} heads of {head_width}")
        if x.dtype == torch.float32:
            if out_dtype != torch.float32:
                raise KernelError("per_head_linear: the float32 product has float32 output")
            out = torch.empty((T, heads, N), dtype=torch.float32, device=x.device)
            self._call("ts_sgemm_nt_batched", _ptr(x), _ptr(w), _ptr(out), T, N, k, x.stride(0), k, heads * N, heads,
                       head_width, N * k, N, _stream())
            return out
        self.calls["library_bmm"] = self.calls.get("library_bmm", 0) + 1
        a = x.view(T, heads, head_width)[:, :, :k].transpose(0, 1)          # [heads, T, k]
        if out_dtype == x.dtype:
            return torch.bmm(a, w.transpose(1, 2)).transpose(0, 1)
        return torch.bmm(a, w.transpose(1, 2), out_dtype=out_dtype).transpose(0, 1)

    def latent_attention(self, q_lat: torch.Tensor, q: torch.Tensor, ctx, binding, heads: int, q_head_width: int,
                         q_rot_offset: int, rank: int, rot: int, freq: torch.Tensor, scale: float, window: int) -> torch.Tensor:
        """
        [T, heads, rank] in q's dtype: per head the softmax-weighted sum of the cached latents, scores
        (q_lat . c + rotated q_rot . k_rot) * scale over the keys the window leaves visible.  q_lat is
        float32 [T, heads, rank] (any token and head strides); the rotated part of the query is read from
        q [T, heads * q_head_width] (rows may be stretches of wider ones) at `q_rot_offset` inside each head and
        rotated here; `rot` 0: there is no such part and `freq` may be None.
        """
        self._check_rows(q, "q")
        if q_lat.dtype != torch.float32 or q_lat.stride(2) != 1 or tuple(q_lat.shape) != (q.shape[0], heads, rank):
            raise KernelError("latent_attention: q_lat must be float32 [T, heads, rank] with unit channel stride")
        if binding.k_pool.dtype != q.dtype:
            raise KernelError(f"cache pool is {binding.k_pool.dtype} but activations are {q.dtype}")
        out = torch.empty((q.shape[0], heads, rank), dtype=q.dtype, device=q.device)
        # the most keys a token of this step sees: bounded by the window and by the longest request (a replayed step: its shape's bound)
        longest = getattr(ctx, "max_ctx_len", None)
        if longest is None:
            longest = int(ctx.positions.max()) + 1
        max_keys = min(window, longest) if window > 0 else longest
        floats = int(self.lib.ts_latent_attention_scratch_floats(q.shape[0], heads, rank, max_keys))
        scratch = None
        if floats:
            store = getattr(ctx, "scratch", None)
            key = ("latent_attention", floats)
            scratch = store.get(key) if store is not None else None
            if scratch is None:
                scratch = torch.empty((floats,), dtype=torch.float32, device=q.device)
                if store is not None:
                    store[key] = scratch
        self._call("ts_latent_attention", _ptr(q_lat), q_lat.stride(0), q_lat.stride(1), _ptr(q), q.stride(0), q_head_width,
                   q_rot_offset, _ptr(freq), _ptr(binding.k_pool), binding.page_stride, binding.entry_offset,
                   binding.page_tokens, binding.num_pages, _ptr(binding.block_table), binding.table_width,
                   _ptr(ctx.positions), _ptr(ctx.seq_of_token), _ptr(out), q.shape[0], heads, rank, rot, scale, window,
                   max_keys, _ptr(scratch), floats, _DTYPE_CODE[q.dtype], _stream())
        if floats:
            self.launches += 1                               # the kernel that merges the splits
        return out

    # ------------------------------------------------------------------ gated activations, routed experts
    GATED_ACTIVATIONS = {"silu": 0, "relu": 1, "clamped_swish": 2, "gelu_tanh": 3}

    def gated_activation(self, gate_up: torch.Tensor, kind: str, limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
        """[T, I] from [T, 2 I] = [gate | up]: silu(g) u, relu(g) u, or the clamped swish g' sigmoid(alpha g') (u' + 1)."""
        if kind == "silu":
            return self.silu_mul(gate_up)
        self._check(gate_up, "gate_up", tuple(_DTYPE_CODE), 2)
        if gate_up.shape[1] % 2 or kind not in self.GATED_ACTIVATIONS:
            raise KernelError(f"gated_activation: kind {kind!r} or odd row width {gate_up.shape[1]}")
        inter = gate_up.shape[1] // 2
        out = torch.empty((gate_up.shape[0], inter), dtype=gate_up.dtype, device=gate_up.device)
        self._call("ts_gated_activation", _ptr(gate_up), _ptr(out), gate_up.shape[0], inter, self.GATED_ACTIVATIONS[kind],
                   limit, alpha, _DTYPE_CODE[gate_up.dtype], _stream())
        return out

    def moe_route(self, logits: torch.Tensor, bias: torch.Tensor | None, ctx, top: int, scoring: str = "softmax_chosen"):
        """
        Routing of one step: (chosen [T, top] int32, share [T, top] float32, offsets [E + 1] int32 of the
        experts' stretches, pair_of_row [T * top], row_of_pair [T * top]).  All on the device; nothing is read back.
        `scoring`: "softmax_chosen" (shares = softmax over the chosen logits) or "sigmoid" (sigmoid of each chosen logit).
        """
        if scoring not in ("softmax_chosen", "sigmoid"):
            raise KernelError(f"moe_route: scoring {scoring!r}")
        self._check(logits, "router logits", torch.float32, 2)
        T, E = logits.shape
        dev = logits.device
        chosen = torch.empty((T, top), dtype=torch.int32, device=dev)
        share = torch.empty((T, top), dtype=torch.float32, device=dev)
        counters = torch.zeros((2 * E,), dtype=torch.int32, device=dev)       # per expert: count, then placement cursor
        offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
        pair_of_row = torch.zeros((T * top,), dtype=torch.int32, device=dev)
        row_of_pair = torch.empty((T * top,), dtype=torch.int32, device=dev)
        seq_of_token = getattr(ctx, "seq_of_token", None)
        self._call("ts_moe_route", _ptr(logits), _ptr(bias), _ptr(seq_of_token), _ptr(chosen), _ptr(share), _ptr(counters),
                   T, E, top, 1 if scoring == "sigmoid" else 0, _stream())
        self._call("ts_moe_arrange", _ptr(chosen), _ptr(counters), counters.data_ptr() + 4 * E, _ptr(offsets),
                   _ptr(pair_of_row), _ptr(row_of_pair), T * top, E, _stream())
        return chosen, share, offsets, pair_of_row, row_of_pair

    def moe_route_grouped(self, logits: torch.Tensor, correction: torch.Tensor | None, ctx, top: int, *, real_experts: int,
                          groups: int = 1, keep: int = 1, weight_scale: float = 1.0, share_eps: float = 0.0):
        """
        Routing by scores that are the softmax over ALL router outputs (logits float32 [T, outputs]): the `top`
        outputs with the largest score + correction among the `keep` best of `groups` groups of neighbours are
        chosen, their shares are the scores divided by their sum + share_eps, times weight_scale.  Outputs from
        `real_experts` on are identity experts.  Returns `moe_route`'s five tensors (an identity choice has
        chosen = -1 and no row; offsets has real_experts + 1 entries) and identity_share [T] float32 (None
        where every output is an expert).
        """
        self._check(logits, "router logits", torch.float32, 2)
        T, outputs = logits.shape
        if correction is not None:
            self._check(correction, "correction", torch.float32, 1)
            if correction.shape[0] != outputs:
                raise KernelError(f"moe_route_grouped: the correction has {correction.shape[0]} elements for {outputs} outputs")
        dev = logits.device
        E = real_experts
        chosen = torch.empty((T, top), dtype=torch.int32, device=dev)
        share = torch.empty((T, top), dtype=torch.float32, device=dev)
        counters = torch.zeros((2 * max(E, 1),), dtype=torch.int32, device=dev)
        offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
        pair_of_row = torch.zeros((T * top,), dtype=torch.int32, device=dev)
        row_of_pair = torch.empty((T * top,), dtype=torch.int32, device=dev)
        identity_share = torch.empty((T,), dtype=torch.float32, device=dev) if E < outputs else None
        self._call("ts_moe_route_grouped", _ptr(logits), _ptr(correction), _ptr(getattr(ctx, "seq_of_token", None)),
                   _ptr(chosen), _ptr(share), _ptr(counters), _ptr(identity_share), T, outputs, E, top, groups, keep,
                   float(weight_scale), float(share_eps), _stream())
        self._call("ts_moe_arrange", _ptr(chosen), _ptr(counters), counters.data_ptr() + 4 * max(E, 1), _ptr(offsets),
                   _ptr(pair_of_row), _ptr(row_of_pair), T * top, E, _stream())
        return chosen, share, offsets, pair_of_row, row_of_pair, identity_share

    def moe_linear(self, x: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, pair_of_row: torch.Tensor | None, top: int,
                   pairs: int, activation: str | None = None, limit: float = 0.0, alpha: float = 1.0,
                   row_scale: torch.Tensor | None = None) -> torch.Tensor:
        """
        [pairs, N] (or [pairs, N / 2] with a gated `activation`): sorted row r of expert e times w[e]^T,
        w [E, N, K].  With `pair_of_row` the input row of sorted row r is x[pair_of_row[r] // top]
        (tokens gathered); without, x[r] (the rows are sorted already).  `activation` "relu2" is ungated:
        relu(s)^2 of the product s, which `row_scale` (float32, one factor a pair) multiplies first.
        """
        unary = 1 if activation == "relu2" else 0
        if unary:
            activation = None
        if row_scale is not None:
            self._check(row_scale, "row scale", torch.float32)
        self._check(x, "x", tuple(_DTYPE_CODE), 2)
        self._check(w, "expert weights", x.dtype, 3)
        E, N, K = w.shape
        if x.shape[1] != K:
            raise KernelError(f"moe_linear: x has {x.shape[1]} columns, the experts {K}")
        gated = activation is not None
        if (x.dtype == torch.bfloat16 and pairs >= self.grouped_mm_min_pairs and K % 8 == 0 and N % 8 == 0
                and hasattr(torch, "_grouped_mm")):
            # many pairs: the library's grouped product (bfloat16 tensor cores, the experts' stretches given on the
            # device), then the gate as a kernel of its own; few pairs and float32 stay on the engine's kernels
            self.calls["library_grouped_mm"] = self.calls.get("library_grouped_mm", 0) + 1
            rows = x if pair_of_row is None else x.index_select(0, torch.div(pair_of_row, top, rounding_mode="floor"))
            full = torch._grouped_mm(rows, w.transpose(1, 2), offs=offsets[1:])
            if unary or row_scale is not None:
                self._call("ts_row_scaled_activation", _ptr(full), _ptr(pair_of_row), _ptr(row_scale), _ptr(full), pairs, N,
                           unary, _DTYPE_CODE[x.dtype], _stream())
                return full
            return self.gated_activation(full, activation, limit, alpha) if gated else full
        out = torch.empty((pairs, N // 2 if gated else N), dtype=x.dtype, device=x.device)
        self._call("ts_moe_linear", _ptr(x), x.stride(0), _ptr(pair_of_row), top, _ptr(offsets), E, _ptr(w), N, K, _ptr(out),
                   pairs, 1 if gated else 0, self.GATED_ACTIVATIONS[activation] if gated else 0, limit, alpha,
                   _ptr(row_scale), unary, _DTYPE_CODE[x.dtype], _stream())
        return out

    def moe_combine(self, y: torch.Tensor, row_of_pair: torch.Tensor, share: torch.Tensor | None,
                    shared_out: torch.Tensor | None, num_tokens: int, x: torch.Tensor | None = None,
                    identity_share: torch.Tensor | None = None) -> torch.Tensor:
        """
        [T, width]: sum over a token's choices of share * y[row of the pair] (share None: 1), plus the shared
        expert's output, plus identity_share[t] * x[t] (the part of experts whose output is their input).
        """
        self._check(y, "y", tuple(_DTYPE_CODE), 2)
        if identity_share is not None:
            self._check(identity_share, "identity share", torch.float32, 1)
            self._check(x, "the experts' input", y.dtype, 2)
            if tuple(x.shape) != (num_tokens, y.shape[1]) or identity_share.shape[0] != num_tokens:
                raise KernelError("moe_combine: the experts' input and the identity shares must have a row a token")
        if shared_out is not None:
            self._check(shared_out, "shared expert output", y.dtype, 2)
        out = torch.empty((num_tokens, y.shape[1]), dtype=y.dtype, device=y.device)
        self._call("ts_moe_combine", _ptr(y), _ptr(row_of_pair), _ptr(share), _ptr(shared_out), _ptr(out), num_tokens,
                   y.shape[1], row_of_pair.shape[0] // max(num_tokens, 1), _DTYPE_CODE[y.dtype],
                   _ptr(x) if identity_share is not None else 0, _ptr(identity_share), _stream())
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

    def linear_unary(self, x: torch.Tensor, weight: torch.Tensor, kind: str, a: float = 0.0, b: float = 0.0) -> torch.Tensor:
        """
        act(x . weight^T) for the activations of `unary_activation`, [M, N]: a few rows of bfloat16 x on the
        weight-streaming kernel with the activation in its epilogue (it reads the product rounded to bfloat16, as
        the separate kernel does, so both ways give the same numbers); else the product and the activation kernel.
        """
        if kind not in self.UNARY_ACTIVATIONS:
            raise KernelError(f"linear_unary: kind {kind!r} of {sorted(self.UNARY_ACTIVATIONS)}")
        self._check(x, "x", tuple(_DTYPE_CODE), 2)
        self._check(weight, "weight", x.dtype, 2)
        if x.shape[1] != weight.shape[1]:
            raise KernelError(f"linear_unary: x has {x.shape[1]} columns, the weight {weight.shape[1]}")
        if not self._skinny(x, weight):
            return self.unary_activation(self.linear(x, weight), kind, a, b)
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        self._call("ts_skinny_linear_unary", _ptr(weight), _ptr(x), _ptr(out), x.shape[0], weight.shape[0], x.shape[1],
                   x.shape[1], weight.shape[0], self.UNARY_ACTIVATIONS[kind], float(a), float(b), _DTYPE_CODE[x.dtype], _stream())
        return out

    def linear_gated(self, x: torch.Tensor, gate_up_weight: torch.Tensor, activation: str, limit: float = 0.0,
                     alpha: float = 1.0) -> torch.Tensor:
        """
        act(x . Wgate^T, x . Wup^T) for the gated activations of `gated_activation`, [M, I], on the same products as
        `linear_swiglu`: the weight-streaming kernel (a few rows) and the tcgen05 kernel (many rows) carry the
        activation in their epilogue; in between, and in float32, the product and the activation kernel.
        """
        if activation == "silu":
            return self.linear_swiglu(x, gate_up_weight)
        self._check(x, "x", tuple(_DTYPE_CODE), 2)
        self._check(gate_up_weight, "weight", x.dtype, 2)
        if gate_up_weight.shape[0] % 2 or x.shape[1] != gate_up_weight.shape[1] or activation not in self.GATED_ACTIVATIONS:
            raise KernelError("linear_gated: the weight must hold gate and up halves over x's columns; activation "
                              f"{activation!r} of {sorted(self.GATED_ACTIVATIONS)}")
        kind = self.GATED_ACTIVATIONS[activation]
        M, K = x.shape
        N = gate_up_weight.shape[0]
        if self._skinny(x, gate_up_weight) and M <= self.swiglu_skinny_rows:
            out = torch.empty((M, N // 2), dtype=x.dtype, device=x.device)
            self._call("ts_skinny_linear_gated", _ptr(gate_up_weight), _ptr(x), _ptr(out), M, N, K, K, N // 2, kind, limit,
                       alpha, _stream())
            return out
        if x.dtype == torch.bfloat16 and M >= self.tcgen05_swiglu_min_rows and self.lib.ts_gemm_tcgen05_supported(
                _ptr(gate_up_weight), _ptr(x), M, N, K, K):
            out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
            self._call("ts_gemm_tcgen05_gated", _ptr(gate_up_weight), _ptr(x), _ptr(out), M, N, K, K, N // 2, kind, limit,
                       alpha, self.error_word().data_ptr(), _stream())
            return out
        return self.gated_activation(self.linear(x, gate_up_weight), activation, limit, alpha)

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
        if (hd * k_pool.dtype.itemsize) % 16:                # rows that are no multiple of 16 bytes: torch's own copy
            k_pool[dst, :, :, :num_slots].copy_(k_pool[src, :, :, :num_slots])
            if v_pool is not None:
                v_pool[dst, :, :, :num_slots].copy_(v_pool[src, :, :, :num_slots])
            return
        self._call("ts_copy_page_slots", _ptr(k_pool), _ptr(v_pool), pages, entries, nkv,
                   page_tokens, hd, k_pool.dtype.itemsize, src, dst,
                   num_slots, _stream())


_OPS: Ops | None = None


def get_ops() -> Ops:
    global _OPS
    if _OPS is None:
        _OPS = Ops()
    return _OPS
