"""Python faces of the CUDA kernels in ``csrc/``.

Each function checks what it is given (device, element type, contiguity,
shapes), launches on torch's current stream and raises ``KernelError`` when the
launcher refuses the arguments or the launch fails.  There is no CPU path: a
tensor that is not on a CUDA device is an error, and so is a missing or
unbuildable extension.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

EPILOGUE_STORE, EPILOGUE_RESIDUAL, EPILOGUE_SILU_MUL = 0, 1, 2
FEW_TOKENS = 32      # up to here a product runs in the few-token kernel, which can also finish q/k/v heads

_REFUSALS = {
    -1: "unsupported element type combination",
    -2: "a size this kernel does not take",
    -3: "a pointer or stride that is not aligned as required",
    -4: "needs more shared memory than the device offers",
}

DEVICE_FAULTS = {
    1: "token id outside the embedding table (token index {d})",
    2: "block table names a page outside the pool (at {d})",
    3: "position outside the rotary table (token index {d})",
    4: "a bounded wait inside a kernel ran out (code {d})",
    5: "row index outside its tensor (row {d})",
}


class KernelError(RuntimeError):
    """A launcher refused its arguments, a launch failed, or a kernel recorded a fault."""


_SIGNATURES = {
    "core": {
        "ls_embed_gather": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "ls_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                       c_float, c_int, c_int64, c_void_p, c_void_p],
        "ls_rmsnorm_shift": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p,
                             c_int, c_int, c_int, c_float, c_void_p],
        "ls_gated_sum": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                         ctypes.c_longlong, c_void_p, c_void_p],
        "ls_clamped_glu": [c_void_p, ctypes.c_longlong, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float,
                           c_void_p, c_void_p, c_int, c_float, c_int, c_void_p],
        "ls_layernorm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
        "ls_norm_merge_add": [c_void_p, c_void_p, c_int, ctypes.c_longlong, c_void_p, c_float, c_void_p, c_int, c_int, c_float,
                              c_float, c_void_p],
        "ls_pair_embed": [c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                          c_int, c_int, ctypes.c_longlong, ctypes.c_longlong, c_float, c_void_p, c_void_p],
        "ls_rows_cast": [c_void_p, c_void_p, c_int, ctypes.c_longlong, c_int, ctypes.c_longlong, c_void_p],
        "ls_scale_cap": [c_void_p, ctypes.c_longlong, c_float, c_float, c_void_p],
        "ls_row_bias": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "ls_weighted_sum": [c_void_p, c_void_p, ctypes.c_longlong, c_int, ctypes.POINTER(c_float), c_void_p, c_int,
                            c_void_p],
        "ls_qk_norm_rope_store": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                  c_void_p, c_void_p],
        "ls_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "ls_gemm_nt_simt": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                            c_int64, c_int64, c_int64, c_int, c_void_p],
        "ls_attention_split_size": [],
        "ls_attention_tile": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                              c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "ls_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                c_void_p, c_void_p, c_void_p, c_void_p],
        "ls_attention_combine": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                 c_void_p, c_void_p],
        "ls_argmax": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "ls_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                      c_int, c_void_p],
    },
}

_SIGNATURES["tc"] = {
    "ls_gemm_tc_token_tile": [c_int, c_int, c_int, c_int],
    "ls_gemm_tc_k_shares": [c_int, c_int],
    "ls_attention_decode_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p],
    "ls_attention_prefill_tc_tile_tokens": [],
    "ls_attention_prefill_tc": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p],
    "ls_gemm_nt_tc_qkv_heads": [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int, c_float, c_void_p,
                                c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "ls_gemm_nt_tc_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int,
                              c_int, c_int, c_int, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p],
    "ls_gemm_nt_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                      c_int, c_void_p, c_void_p],
}

_SIGNATURES["seq"] = {
    "ls_qkv_finish": [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                      c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p],
    "ls_latent_finish": [c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                         c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_int, c_float, c_void_p, c_void_p, c_void_p],
    "ls_heads_product": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_void_p],
    "ls_sigmoid_power_decay": [c_void_p, c_void_p, ctypes.c_longlong, c_int, c_float, c_void_p],
    "ls_find_portions": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p],
    "ls_delta_prep": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                      c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "ls_double_exp_decay": [c_void_p, c_void_p, ctypes.c_longlong, c_int, c_void_p],
    "ls_shift_mix": [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int, c_int,
                     c_void_p],
    "ls_state_rule": [c_int, c_int, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_int64, c_float, c_int64, c_void_p],
    "ls_unit_gates": [c_void_p, ctypes.c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_longlong,
                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                      c_int, c_float, c_void_p],
    "ls_unit_scan": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int, c_int, c_void_p,
                     c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_int, c_void_p],
    "ls_rotate_rows": [c_void_p, ctypes.c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "ls_head_rms_gate": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_float, c_int64, c_void_p],
    "ls_tanh_rows": [c_void_p, c_int, ctypes.c_longlong, c_void_p],
    "ls_experts_tile_rows": [],
    "ls_experts_route": [c_void_p, ctypes.c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "ls_experts_mix": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                       ctypes.c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "ls_experts_plan": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_void_p],
    "ls_experts_route_plan": [c_void_p, ctypes.c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                              c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "ls_experts_tc_tile_rows": [],
    "ls_experts_gather": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ls_experts_product_tc": [c_int, c_void_p, c_int, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_void_p,
                              c_int, c_int, c_void_p, c_void_p],
    "ls_experts_product": [c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                           c_int, c_void_p],
    "ls_experts_combine": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
}

_libs: dict[str, ctypes.CDLL] = {}


def library(name: str = "core") -> ctypes.CDLL:
    """The loaded extension library `name` (compiled at first use)."""
    lib = _libs.get(name)
    if lib is None:
        lib = _build.load(name)
        for fn, argtypes in _SIGNATURES.get(name, {}).items():
            f = getattr(lib, fn)
            f.argtypes = argtypes
            f.restype = c_int
        _libs[name] = lib
    return lib


def set_gemm_tc_pairs(on: bool) -> None:
    """Whether tensor-core products of more than 128 tokens run on pairs of blocks that share
    a tile of 256 tokens (tcgen05 cta_group::2; the default) or on single blocks with tiles of
    128 tokens.  The sums are the same either way."""
    fn = library("tc").ls_set_gemm_tc_pairs
    fn.argtypes, fn.restype = [c_int], None
    fn(1 if on else 0)


def set_attention_prefill_pairs(mode: int) -> None:
    """How the tensor-core attention of prompt portions takes the heads of a key head: 0 one
    head a block; 1 (the default) two heads a block, sharing the key and value tiles, where the
    group size is even and the items fill the device twice over; 2 wherever the group is even."""
    fn = library("tc").ls_set_attention_prefill_pairs
    fn.argtypes, fn.restype = [c_int], None
    fn(int(mode))


def set_dependent_launch(on: bool) -> None:
    """Programmatic dependent launch of all kernels (on by default): a kernel is
    scheduled while its predecessor drains and waits for it before it touches memory."""
    for name in ["core", "tc"] + [n for n in _libs if n not in ("core", "tc")]:
        fn = getattr(library(name), f"ls_set_dependent_launch_{name}")
        fn.argtypes, fn.restype = [c_int], None
        fn(1 if on else 0)


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError(
            "lockstep_b200 runs on a CUDA device only (sm_100a); there is no CPU fallback")


def _stream() -> int:
    """The current stream's handle (also while a graph is being captured).  Asked of torch's
    C layer directly: ``torch.cuda.current_stream()`` builds a Python object on every call,
    which was a third of the host's share of a step."""
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 or bfloat16)") from None


def _dev(t: torch.Tensor, name: str, dtype=None) -> int:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device; there is no CPU fallback")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _opt(t, name, dtype=None) -> int:
    return 0 if t is None else _dev(t, name, dtype)


# bfloat16 work goes to the tensor cores unless this is cleared (a debugging aid)
USE_TENSOR_CORES = [True]

# kernel launches since the counter was last cleared: launcher calls (each is at
# least one kernel) plus, for a replayed graph, the calls that were recorded in it
LAUNCHES = [0]


def kernel_counts() -> dict[str, int]:
    """How often each kernel's launcher has launched in this process (a launch recorded into
    a graph counts once, its replays do not), over the libraries that are loaded."""
    out: dict[str, int] = {}
    library("core")
    for name, lib in list(_libs.items()):
        names_fn = getattr(lib, f"ls_kernel_names_{name}")
        names_fn.restype, names_fn.argtypes = ctypes.c_char_p, []
        names = names_fn().decode("ascii").split(",")
        counts = (ctypes.c_ulonglong * len(names))()
        fn = getattr(lib, f"ls_kernel_launches_{name}")
        fn.restype, fn.argtypes = c_int, [ctypes.POINTER(ctypes.c_ulonglong), c_int]
        fn(counts, len(names))
        for kernel, count in zip(names, counts):
            out[kernel] = out.get(kernel, 0) + int(count)
    return out


def _check(status: int, what: str) -> None:
    if status == 0:
        LAUNCHES[0] += 1
        return
    if status < 0:
        raise KernelError(f"{what}: {_REFUSALS.get(status, f'refused with code {status}')}")
    raise KernelError(f"{what}: CUDA launch failed with error {status}")


def new_error_word(device) -> torch.Tensor:
    """Two int32 on the device: the first fault a kernel recorded and its detail."""
    return torch.zeros(2, dtype=torch.int32, device=device)


def raise_on_fault(err: torch.Tensor) -> None:
    """Read the error word (synchronises) and raise if a kernel recorded a fault."""
    code, detail = err.tolist()
    if code != 0:
        err.zero_()
        raise KernelError("device fault: " + DEVICE_FAULTS.get(code, "code {d}").format(d=detail))


# ---------------------------------------------------------------------------

def attention_split_size() -> int:
    return int(library().ls_attention_split_size())


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor,
                 accumulate: bool = False) -> None:
    """out[t] = table[ids[t]] (float32), or out[t] += table[ids[t]] with ``accumulate``."""
    tokens, width = out.shape
    if ids.numel() != tokens or table.shape[1] != width:
        raise KernelError("embed_gather: shapes do not agree")
    _check(library().ls_embed_gather(
        _dev(ids, "ids", torch.int32), _dev(table, "table"), _code(table),
        _dev(out, "out", torch.float32), tokens, width, table.shape[0], 1 if accumulate else 0,
        _dev(err, "err", torch.int32), _stream()), "embed_gather")


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, out: torch.Tensor, eps: float, err: torch.Tensor,
            row_index: torch.Tensor | None = None, groups: int = 1, columns: int | None = None) -> None:
    """``groups`` > 1: a row is cut into that many equal consecutive parts, each divided by its
    own root mean square; the gain runs over the whole row.  ``columns``: only the first so many
    columns of every row of ``x`` are the row to norm (a part of a wider product's result)."""
    rows, width = out.shape
    if groups < 1 or width % groups:
        raise KernelError(f"rmsnorm: a row of {width} elements cannot be cut into {groups} equal parts")
    if columns is not None and (columns != width or x.shape[1] < width):
        raise KernelError("rmsnorm: the columns to norm do not match the output")
    if (columns is None and x.shape[1] != width) or gain.numel() != width:
        raise KernelError("rmsnorm: shapes do not agree")
    if row_index is None and x.shape[0] != rows:
        raise KernelError("rmsnorm: row counts do not agree")
    if row_index is not None and row_index.numel() != rows:
        raise KernelError("rmsnorm: row_index does not match the output rows")
    _check(library().ls_rmsnorm(
        _dev(x, "x", torch.float32), _opt(row_index, "row_index", torch.int32), _dev(gain, "gain"),
        _code(gain), _dev(out, "out"), _code(out), rows, width, x.shape[0], float(eps), int(groups), x.shape[1],
        _dev(err, "err", torch.int32), _stream()), "rmsnorm")


def rmsnorm_shift(h, gain, eps: float, mu, state, token_slot, y, x) -> None:
    """y = rmsnorm(h) (``gain`` per column) and x[t] = y[t] + (y[t - 1] - y[t]) * mu in one pass, the row before a
    portion's first one taken from ``state[slot]`` (float32 [slots, >= width]); bit for bit what ``rmsnorm``
    followed by ``shift_mix`` gives.  ``h`` float32 [tokens, width]; ``y`` and ``x`` of one element type."""
    tokens, width = h.shape
    if y.shape != h.shape or x.shape != h.shape or y.dtype != x.dtype or gain.numel() != width or mu.numel() != width:
        raise KernelError("rmsnorm_shift: shapes do not agree")
    if state.dim() != 2 or state.shape[1] < width or token_slot.numel() != tokens:
        raise KernelError("rmsnorm_shift: the carried rows do not match")
    _check(library().ls_rmsnorm_shift(
        _dev(h, "h", torch.float32), _dev(gain, "gain"), _code(gain), _dev(mu, "mu", torch.float32),
        _dev(state, "state", torch.float32), state.stride(0), _dev(token_slot, "token_slot", torch.int32),
        _dev(y, "y"), _dev(x, "x"), _code(y), tokens, width, float(eps), _stream()), "rmsnorm_shift")


def gated_sum(residual, branches, z, bias, carry=None) -> None:
    """residual += sum_b sigmoid(z[:, b] + bias[b]) * branches[b]: ``branches`` float32 [n, tokens, width], ``z``
    float32 [tokens, n * width] and ``bias`` float32 [n * width], or both None for a plain sum.  ``carry`` =
    (y [tokens, width], state float32 [slots, >= width], token_slot): the row of y of every token that ends its
    request's portion is kept in ``state[slot]``."""
    n, tokens, width = branches.shape
    if tuple(residual.shape) != (tokens, width) or (z is None) != (bias is None):
        raise KernelError("gated_sum: shapes do not agree")
    if z is not None and (tuple(z.shape) != (tokens, n * width) or bias.numel() != n * width):
        raise KernelError("gated_sum: the gates do not match the branches")
    y, state, token_slot = carry if carry is not None else (None, None, None)
    if y is not None and (tuple(y.shape) != (tokens, width) or state.dim() != 2 or state.shape[1] < width
                          or token_slot.numel() != tokens):
        raise KernelError("gated_sum: the rows to carry do not match")
    _check(library().ls_gated_sum(
        _dev(residual, "residual", torch.float32), _dev(branches, "branches", torch.float32), n,
        _opt(z, "z", torch.float32), _opt(bias, "bias", torch.float32), tokens, width, _opt(y, "y"),
        _code(y) if y is not None else F32, _opt(state, "state", torch.float32),
        state.stride(0) if state is not None else 0, _opt(token_slot, "token_slot", torch.int32), _stream()), "gated_sum")


def qk_norm_rope_store(qkv, q_out, pages, q_gain, k_gain, cos, sin, positions, token_req,
                       block_table, nq: int, nkv: int, d: int, rot_dim: int, eps: float,
                       write_cache: bool, err, interleaved: bool = False) -> None:
    """pages: [num_pages, 2, nkv, page_size, d] of one cache layer (may be None if not written).
    ``interleaved``: a rotated pair is elements (2i, 2i + 1) of the head instead of
    (i, i + rot_dim / 2)."""
    tokens = qkv.shape[0]
    if qkv.shape[1] != (nq + 2 * nkv) * d or q_out.shape != (tokens, nq * d):
        raise KernelError("qk_norm_rope_store: shapes do not agree")
    if (q_gain is None) != (k_gain is None):
        raise KernelError("qk_norm_rope_store: q and k gains come together")
    if write_cache:
        if pages.dtype != qkv.dtype or pages.shape[1:3] != (2, nkv) or pages.shape[4] != d:
            raise KernelError("qk_norm_rope_store: cache pages do not match the projections")
        num_pages, page_size = pages.shape[0], pages.shape[3]
    else:
        num_pages, page_size = 0, 1
    half = rot_dim // 2
    if rot_dim:
        if cos.shape != sin.shape or cos.shape[1] != half:
            raise KernelError("qk_norm_rope_store: rotary tables do not match rot_dim")
    gain_code = _code(q_gain) if q_gain is not None else F32
    if q_gain is not None and (q_gain.dtype != k_gain.dtype or q_gain.numel() != d or k_gain.numel() != d):
        raise KernelError("qk_norm_rope_store: gains do not match the head size")
    _check(library().ls_qk_norm_rope_store(
        _dev(qkv, "qkv"), _dev(q_out, "q_out", qkv.dtype), _opt(pages if write_cache else None, "pages"),
        _code(qkv), _opt(q_gain, "q_gain"), _opt(k_gain, "k_gain"), gain_code,
        _opt(cos if rot_dim else None, "cos", torch.float32),
        _opt(sin if rot_dim else None, "sin", torch.float32),
        _dev(positions, "positions", torch.int32), _dev(token_req, "token_req", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[-1], tokens, nq, nkv, d,
        rot_dim, page_size, num_pages, cos.shape[0] if rot_dim else 0, float(eps),
        1 if write_cache else 0, 1 if interleaved else 0, _dev(err, "err", torch.int32), _stream()),
        "qk_norm_rope_store")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    rows, width = out.shape
    if gate_up.shape != (rows, 2 * width) or gate_up.dtype != out.dtype:
        raise KernelError("silu_mul: shapes do not agree")
    _check(library().ls_silu_mul(_dev(gate_up, "gate_up"), _dev(out, "out"), _code(out), rows, width,
                                 _stream()), "silu_mul")


def clamped_glu(gate_up, bias, out, limit: float, alpha: float, residual=None, residual_bias=None,
                up_offset: float = 1.0, gelu: bool = False) -> None:
    """(``up_offset``: what is added to u, 1 unless given; ``gelu``: the tanh form of gelu of g in place of g sigmoid(alpha g).)
    out = g sigmoid(alpha g) (u + 1) with g = min(gate + b, limit), u = clamp(up + b, -limit, limit), from
    ``gate_up`` [rows, 2 width] (gate columns, then up columns; float32 or the type of ``out``; a view of some
    columns of a wider tensor is fine) and ``bias`` [2 width] or None.  With ``residual`` (float32 [rows, w]) and ``residual_bias`` [w] the same launch adds the
    bias of the projection that follows into the residual stream."""
    rows, width = out.shape
    if gate_up.shape != (rows, 2 * width) or (bias is not None and bias.numel() != 2 * width):
        raise KernelError("clamped_glu: shapes do not agree")
    if (residual is None) != (residual_bias is None) or \
            (residual is not None and (residual.shape[0] != rows or residual_bias.numel() != residual.shape[1])):
        raise KernelError("clamped_glu: the residual stream and its bias do not agree")
    if bias is not None and residual_bias is not None and bias.dtype != residual_bias.dtype:
        raise KernelError("clamped_glu: biases of two element types")
    some = bias if bias is not None else residual_bias
    gp, g_ld = _rows(gate_up, "gate_up")
    _check(library().ls_clamped_glu(
        gp, g_ld, _code(gate_up), _opt(bias, "bias"), _code(some) if some is not None else F32,
        _dev(out, "out"), _code(out), rows, width, float(limit), float(alpha), _opt(residual, "residual", torch.float32),
        _opt(residual_bias, "residual_bias"), residual.shape[1] if residual is not None else 0, float(up_offset),
        1 if gelu else 0, _stream()), "clamped_glu")


def row_bias(x, bias, add: bool = False) -> None:
    """Every row of ``x`` (float32 [rows, width]) set to ``bias`` (to zero for None), or ``bias`` added to it."""
    rows, width = x.shape
    if bias is not None and bias.numel() != width:
        raise KernelError("row_bias: the bias does not match the rows")
    _check(library().ls_row_bias(_dev(x, "x", torch.float32), _opt(bias, "bias"), _code(bias) if bias is not None else F32,
                                 rows, width, 1 if add else 0, _stream()), "row_bias")


def weighted_sum(residual, branches, scales, bias=None) -> None:
    """residual += sum_b scales[b] * branches[b] (+ bias); ``branches`` float32 [n, *residual.shape], ``bias``
    float32 [residual.shape[-1]] or None."""
    n = branches.shape[0]
    if tuple(branches.shape[1:]) != tuple(residual.shape) or len(scales) != n:
        raise KernelError("weighted_sum: shapes do not agree")
    if bias is not None and bias.numel() != residual.shape[-1]:
        raise KernelError("weighted_sum: the bias does not match the rows")
    _check(library().ls_weighted_sum(_dev(residual, "residual", torch.float32), _dev(branches, "branches", torch.float32),
                                     residual.numel(), n, (c_float * n)(*[float(v) for v in scales]),
                                     _opt(bias, "bias", torch.float32), residual.shape[-1], _stream()), "weighted_sum")


def layernorm(x, gain, out, eps: float, err, row_index=None) -> None:
    """out = (x - mean) rsqrt(var + eps) gain over float32 rows of ``x`` (all, or those ``row_index`` names)."""
    rows, width = out.shape
    if x.shape[1] != width or gain.numel() != width or (row_index is None and x.shape[0] != rows) \
            or (row_index is not None and row_index.numel() != rows):
        raise KernelError("layernorm: shapes do not agree")
    _check(library().ls_layernorm(
        _dev(x, "x", torch.float32), _opt(row_index, "row_index", torch.int32), _dev(gain, "gain"), _code(gain),
        _dev(out, "out"), _code(out), rows, width, x.shape[0], float(eps), _dev(err, "err", torch.int32), _stream()), "layernorm")


def norm_merge_add(residual, branches, branch_gain, scale: float, post_gain, eps_branch: float, eps_post: float) -> None:
    """residual += post(scale sum_b rms(branches[b]) branch_gain[b]): ``branches`` float32 [n, rows, width]; with
    ``branch_gain`` (float32 [n, width]) every branch is divided by its root mean square and multiplied by its gain,
    without it the branches are summed as they are; ``post_gain`` (float32 [width]): the sum goes through a layer norm
    with this gain before it is added."""
    n, rows, width = branches.shape
    if tuple(residual.shape) != (rows, width) or (branch_gain is not None and tuple(branch_gain.shape) != (n, width)) \
            or (post_gain is not None and post_gain.numel() != width):
        raise KernelError("norm_merge_add: shapes do not agree")
    _check(library().ls_norm_merge_add(
        _dev(residual, "residual", torch.float32), _dev(branches, "branches", torch.float32), n, rows * width,
        _opt(branch_gain, "branch_gain", torch.float32), float(scale), _opt(post_gain, "post_gain", torch.float32),
        rows, width, float(eps_branch), float(eps_post), _stream()), "norm_merge_add")


def pair_embed(ids, token_slot, carried, table, pairs, out, factor: float, mul_prev: int, mul_cur: int, err) -> None:
    """out[t] = table[ids[t]] factor + pairs[(previous id x mul_prev + ids[t] x mul_cur) mod buckets], the last row of
    ``pairs`` [buckets + 1, width] for a request's first token; the previous id is the token in front where it belongs to
    the same request, else what ``carried`` (int32 [slots, >= 1]: last token + 1) holds, which is then brought up to date.
    Without ``pairs``: the scaled gather alone."""
    tokens, width = out.shape
    if ids.numel() != tokens or table.shape[1] != width or (pairs is not None and (pairs.shape[1] != width or pairs.dtype != table.dtype)):
        raise KernelError("pair_embed: shapes do not agree")
    _check(library().ls_pair_embed(
        _dev(ids, "ids", torch.int32), _opt(token_slot, "token_slot", torch.int32), _opt(carried, "carried", torch.int32),
        carried.stride(0) if carried is not None else 0, _dev(table, "table"), _opt(pairs, "pairs"), _code(table),
        _dev(out, "out", torch.float32), tokens, width, table.shape[0], pairs.shape[0] - 1 if pairs is not None else 0,
        int(mul_prev), int(mul_cur), float(factor), _dev(err, "err", torch.int32), _stream()), "pair_embed")


def rows_cast(src, dst) -> None:
    """dst = src (float32 [rows, width]) in the type of ``dst``, which may be some columns of a wider tensor."""
    if src.shape != dst.shape:
        raise KernelError("rows_cast: shapes do not agree")
    dp, ld = _rows(dst, "dst")
    _check(library().ls_rows_cast(_dev(src, "src", torch.float32), dp, _code(dst), src.shape[0], src.shape[1], ld, _stream()),
           "rows_cast")


def scale_cap(x, factor: float, cap: float) -> None:
    """x <- x factor, then cap tanh(x / cap) where cap > 0; float32, in place."""
    _check(library().ls_scale_cap(_dev(x, "x", torch.float32), x.numel(), float(factor), float(cap), _stream()), "scale_cap")


def _rows(t: torch.Tensor, name: str) -> tuple[int, int]:
    """(pointer, row pitch in elements) of a 2-D operand whose rows are contiguous: a whole
    tensor, or a view of some columns of one."""
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device; there is no CPU fallback")
    if t.dim() != 2 or t.stride(1) != 1 or (t.shape[0] > 1 and t.stride(0) < t.shape[1]):
        raise KernelError(f"{name} must be two-dimensional with contiguous rows")
    # (a single row's stride says nothing about the rows; a view of a wider row keeps its pitch)
    return t.data_ptr(), (t.stride(0) if t.stride(0) >= t.shape[1] else t.shape[1])


def gemm_nt_simt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE) -> None:
    """c = a @ w.T on the CUDA cores with the chosen epilogue (see csrc/gemm_simt.cu).  ``a`` may
    be a view of some columns of a wider tensor."""
    m, k = a.shape
    n = c.shape[1]
    rows_w = 2 * n if epilogue == EPILOGUE_SILU_MUL else n
    if w.shape != (rows_w, k) or c.shape[0] != m or a.dtype != w.dtype:
        raise KernelError(f"gemm_nt: shapes do not agree: a {tuple(a.shape)} w {tuple(w.shape)} c {tuple(c.shape)}")
    ap, lda = _rows(a, "a")
    _check(library().ls_gemm_nt_simt(
        ap, _dev(w, "w"), _dev(c, "c"), _code(a), _code(c), m, n, k, lda, k, n, epilogue,
        _stream()), "gemm_nt_simt")


def _slopes(slopes, nq: int) -> int:
    if slopes is not None and slopes.numel() != nq:
        raise KernelError(f"a score bias needs one slope per query head: {slopes.numel()} for {nq} heads")
    return _opt(slopes, "slopes", torch.float32)


def attention_tile(q, pages, out, part_acc, part_ml, work, n_work, block_table, nq, nkv, d,
                   window, scale, err, slopes=None, log_rates=None, sinks=None, softcap: float = 0.0) -> None:
    """``window`` > 0: a query reads the last ``window`` positions; < 0: the positions of its own chunk of
    ``-window`` positions, chunks counted from position 0; 0: every earlier position.  ``softcap`` > 0: the scaled
    score becomes softcap tanh(score / softcap) before any bias.  ``slopes`` (float32 [nq] or None): slopes[head] x (key position - query position) is added
    to every score; with ``log_rates`` [nq] as well, slopes[head] x ln(1 + log_rates[head] x (query
    position - key position)) is taken off instead.  ``sinks`` [nq]: exp(sinks[head]) is one more
    term of the softmax's denominator (rows that write ``out``; partials get theirs in
    ``attention_combine``)."""
    _check(library().ls_attention_tile(
        _dev(q, "q"), _dev(pages, "pages", q.dtype), _opt(out, "out", q.dtype),
        _opt(part_acc, "part_acc", torch.float32), _opt(part_ml, "part_ml", torch.float32), _code(q),
        _dev(work, "work", torch.int32), n_work, _dev(block_table, "block_table", torch.int32),
        block_table.shape[-1], nq, nkv, d, pages.shape[3], pages.shape[0], int(window), float(scale), float(softcap),
        _slopes(slopes, nq), _slopes(log_rates, nq), _slopes(sinks, nq), _dev(err, "err", torch.int32),
        _stream()), "attention_tile")


def attention_decode(q, pages, part_acc, part_ml, work, n_work, block_table, nq, nkv, d, window,
                     scale, err, slopes=None, log_rates=None, softcap: float = 0.0) -> bool:
    """Returns False (and launches nothing) for shapes the decode kernel does not take."""
    status = library().ls_attention_decode(
        _dev(q, "q"), _dev(pages, "pages", q.dtype), _dev(part_acc, "part_acc", torch.float32),
        _dev(part_ml, "part_ml", torch.float32), _code(q), _dev(work, "work", torch.int32), n_work,
        _dev(block_table, "block_table", torch.int32), block_table.shape[-1], nq, nkv, d,
        pages.shape[3], pages.shape[0], int(window), float(scale), float(softcap), _slopes(slopes, nq),
        _slopes(log_rates, nq), _dev(err, "err", torch.int32), _stream())
    if status == -2:
        return False
    _check(status, "attention_decode")
    return True


def attention_decode_mma(q, pages, part_acc, part_ml, work, n_work, block_table, nq, nkv, d, window,
                         scale, err, slopes=None, log_rates=None) -> bool:
    """Decode attention on mma.sync with TMA-fed pages (csrc/attention_decode_mma.cu): bfloat16,
    head size 64 or 128, groups up to 16; ``slopes`` and ``log_rates`` together: the bias that grows
    with the logarithm of the distance (see ``attention_tile``).  Returns False (nothing launched)
    otherwise."""
    if (slopes is None) != (log_rates is None):
        return False
    if q.dtype != torch.bfloat16 or not USE_TENSOR_CORES[0]:
        return False
    status = library("tc").ls_attention_decode_mma(
        _dev(q, "q"), _dev(pages, "pages", q.dtype), _dev(part_acc, "part_acc", torch.float32),
        _dev(part_ml, "part_ml", torch.float32), _dev(work, "work", torch.int32), n_work,
        _dev(block_table, "block_table", torch.int32), block_table.shape[-1], nq, nkv, d,
        pages.shape[3], pages.shape[0], int(window), float(scale), _slopes(slopes, nq), _slopes(log_rates, nq),
        _dev(err, "err", torch.int32), _stream())
    if status == -2:
        return False
    _check(status, "attention_decode_mma")
    return True


def attention_prefill_tc_tile_tokens() -> int:
    return int(library("tc").ls_attention_prefill_tc_tile_tokens())


def attention_prefill_tc(q, pages, out, work, n_work, block_table, nq, nkv, d, window, scale, err,
                         slopes=None, log_rates=None, sinks=None, softcap: float = 0.0) -> bool:
    """Attention of prompt portions on tcgen05 (csrc/attention_prefill_tc.cu): bfloat16, head
    size 64 or 128, work items of up to 128 tokens; ``slopes`` with ``log_rates`` (the bias that
    grows with the logarithm of the distance), ``slopes`` alone (the bias linear in the distance), ``softcap`` and
    ``sinks`` as in ``attention_tile``.  Returns False (nothing launched) for anything else."""
    if log_rates is not None and (slopes is None or softcap):
        return False
    if q.dtype != torch.bfloat16 or not USE_TENSOR_CORES[0]:
        return False
    status = library("tc").ls_attention_prefill_tc(
        _dev(q, "q"), _dev(pages, "pages", q.dtype), _dev(out, "out", q.dtype), q.shape[0],
        _dev(work, "work", torch.int32), n_work, _dev(block_table, "block_table", torch.int32),
        block_table.shape[-1], nq, nkv, d, pages.shape[3], pages.shape[0], int(window), float(scale),
        _slopes(slopes, nq), _slopes(log_rates, nq), _slopes(sinks, nq), float(softcap), _dev(err, "err", torch.int32), _stream())
    if status in (-2, -3):
        return False
    _check(status, "attention_prefill_tc")
    return True


def attention_combine(part_acc, part_ml, out, items, n_items, nq, d, sinks=None) -> None:
    _check(library().ls_attention_combine(
        _dev(part_acc, "part_acc", torch.float32), _dev(part_ml, "part_ml", torch.float32),
        _dev(out, "out"), _code(out), _dev(items, "items", torch.int32), n_items, nq, d, _slopes(sinks, nq),
        _stream()), "attention_combine")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    rows, vocab = logits.shape
    scratch = torch.empty(rows * 128, dtype=torch.int32, device=logits.device)
    _check(library().ls_argmax(_dev(logits, "logits", torch.float32), _dev(out, "out", torch.int32),
                               _dev(scratch, "scratch"), rows, vocab, _stream()), "argmax")


def sample_scratch_floats(rows: int, vocab: int) -> int:
    """Floats of scratch ``sample`` needs for ``rows`` rows of ``vocab`` logits (0: none)."""
    fn = library().ls_sample_scratch_floats
    fn.argtypes, fn.restype = [c_int, c_int], ctypes.c_longlong
    return int(fn(rows, vocab))


def sample(logits, probs, temperature, top_p, keys, positions, out) -> None:
    """keys, positions: [rows, 2] int32 holding the low and high 32 bits.  ``probs``: float32
    scratch of ``sample_scratch_floats(rows, vocab)`` elements, or None where that is 0."""
    rows, vocab = logits.shape
    if probs is not None and probs.numel() < rows * vocab:
        raise KernelError("sample: probs scratch does not match the logits")
    if probs is None and sample_scratch_floats(rows, vocab):
        raise KernelError("sample: this vocabulary needs a scratch for the probabilities")
    _check(library().ls_sample(
        _dev(logits, "logits", torch.float32), _opt(probs, "probs", torch.float32),
        _dev(temperature, "temperature", torch.float32), _dev(top_p, "top_p", torch.float32),
        _dev(keys, "keys", torch.int32), _dev(positions, "positions", torch.int32),
        _dev(out, "out", torch.int32), rows, vocab, _stream()), "sample")



def gemm_nt_tc(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int, err: torch.Tensor) -> bool:
    """c = a @ w.T on the tcgen05 tensor cores (csrc/gemm_tc.cu).  Returns False,
    having launched nothing, when TMA cannot address the operands (a row pitch
    that is no multiple of 16 bytes): the caller then uses the CUDA-core product."""
    m, k = a.shape
    n = c.shape[1]
    rows_w = 2 * n if epilogue == EPILOGUE_SILU_MUL else n
    if w.shape != (rows_w, k) or c.shape[0] != m or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_nt_tc: shapes or types do not agree: a {tuple(a.shape)} w {tuple(w.shape)} c {tuple(c.shape)}")
    ap, lda = _rows(a, "a")
    status = library("tc").ls_gemm_nt_tc(
        ap, _dev(w, "w"), _dev(c, "c"), _code(c), m, n, k, lda, k, n, epilogue,
        _dev(err, "err", torch.int32), _stream())
    if status in (-2, -3):
        return False
    _check(status, "gemm_nt_tc")
    return True


def gemm_nt_tc_rmsnorm(h: torch.Tensor, gain: torch.Tensor, eps: float, w: torch.Tensor, c: torch.Tensor,
                       epilogue: int, err: torch.Tensor, row_index: torch.Tensor | None = None, groups: int = 1) -> bool:
    """c = rmsnorm(h)[rows] @ w.T with the norm made inside the product's kernel, bit for bit
    what ``rmsnorm`` (in ``groups`` parts) followed by ``gemm_nt_tc`` gives.  h [rows, k] float32, w bfloat16.
    Returns False, having launched nothing, where the fused form does not apply (many
    tokens, a weight whose depth is not shared out, unaligned rows)."""
    if not USE_TENSOR_CORES[0] or w.dtype != torch.bfloat16:
        return False
    k = h.shape[1]
    m, n = c.shape
    rows_w = 2 * n if epilogue == EPILOGUE_SILU_MUL else n
    if w.shape != (rows_w, k) or gain.numel() != k:
        raise KernelError("gemm_nt_tc_rmsnorm: shapes do not agree")
    if row_index is None and h.shape[0] != m:
        raise KernelError("gemm_nt_tc_rmsnorm: row counts do not agree")
    status = library("tc").ls_gemm_nt_tc_rmsnorm(
        _dev(h, "h", torch.float32), _opt(row_index, "row_index", torch.int32), h.shape[0],
        _dev(gain, "gain"), _code(gain), float(eps), _dev(w, "w"), _dev(c, "c"), _code(c), m, n, k, k, n,
        epilogue, int(groups), _dev(err, "err", torch.int32), _stream())
    if status in (-2, -3):
        return False
    _check(status, "gemm_nt_tc_rmsnorm")
    return True


def gemm_nt_tc_qkv_heads(x, w, q_out, pages, q_gain, k_gain, cos, sin, positions, token_req, block_table,
                         nq: int, nkv: int, d: int, rot_dim: int, head_eps: float, write_cache: bool, err,
                         normed=None) -> bool:
    """The q/k/v projection of few tokens with the work of ``qk_norm_rope_store`` done in the
    product's epilogue (same bits, one kernel).  ``x`` [tokens, k] bfloat16, or None with
    ``normed`` = (h float32 [rows, k], gain, eps, row_index or None) to make the RMSNorm of the
    rows inside the product as well.  Returns False, having launched nothing, where the fused
    form does not apply; the caller then runs the product and ``qk_norm_rope_store``."""
    if not USE_TENSOR_CORES[0] or w.dtype != torch.bfloat16 or q_out.dtype != torch.bfloat16:
        return False
    tokens = q_out.shape[0]
    k = w.shape[1]
    if w.shape[0] != (nq + 2 * nkv) * d or q_out.shape != (tokens, nq * d):
        raise KernelError("gemm_nt_tc_qkv_heads: shapes do not agree")
    if (q_gain is None) != (k_gain is None):
        raise KernelError("gemm_nt_tc_qkv_heads: q and k gains come together")
    if q_gain is not None and (q_gain.dtype != k_gain.dtype or q_gain.numel() != d or k_gain.numel() != d):
        raise KernelError("gemm_nt_tc_qkv_heads: gains do not match the head size")
    if write_cache:
        if pages.dtype != torch.bfloat16 or pages.shape[1:3] != (2, nkv) or pages.shape[4] != d:
            raise KernelError("gemm_nt_tc_qkv_heads: cache pages do not match the projections")
        num_pages, page_size = pages.shape[0], pages.shape[3]
    else:
        num_pages, page_size = 0, 1
    if rot_dim and (cos.shape != sin.shape or cos.shape[1] != rot_dim // 2):
        raise KernelError("gemm_nt_tc_qkv_heads: rotary tables do not match rot_dim")
    if normed is None:
        if x.dtype != torch.bfloat16 or x.shape != (tokens, k):
            raise KernelError("gemm_nt_tc_qkv_heads: the token operand does not match")
        xp, ldx, hp, rows_p, src_rows, gain_p, gain_code, eps = _dev(x, "x"), k, None, None, 0, None, F32, 0.0
    else:
        h, gain, eps, row_index = normed
        if h.shape[1] != k or gain.numel() != k or (row_index is None and h.shape[0] != tokens):
            raise KernelError("gemm_nt_tc_qkv_heads: the rows to norm do not match")
        xp, ldx, hp, rows_p = None, 0, _dev(h, "h", torch.float32), _opt(row_index, "row_index", torch.int32)
        src_rows, gain_p, gain_code = h.shape[0], _dev(gain, "gain"), _code(gain)
    status = library("tc").ls_gemm_nt_tc_qkv_heads(
        xp, ldx, hp, rows_p, src_rows, gain_p, gain_code, float(eps), _dev(w, "w"), k, tokens, k,
        _dev(q_out, "q_out"), _opt(pages if write_cache else None, "pages"), _opt(q_gain, "q_gain"),
        _opt(k_gain, "k_gain"), _code(q_gain) if q_gain is not None else F32,
        _opt(cos if rot_dim else None, "cos", torch.float32), _opt(sin if rot_dim else None, "sin", torch.float32),
        _dev(positions, "positions", torch.int32), _dev(token_req, "token_req", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[-1], nq, nkv, d, rot_dim, page_size,
        num_pages, cos.shape[0] if rot_dim else 0, float(head_eps), 1 if write_cache else 0,
        _dev(err, "err", torch.int32), _stream())
    if status in (-2, -3):
        return False
    _check(status, "gemm_nt_tc_qkv_heads")
    return True


_tc_err: dict = {}


def gemm_nt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE,
            err: torch.Tensor | None = None) -> None:
    """c = a @ w.T with float32 accumulation and the chosen epilogue.

    a [m, k] and w [n, k] (or [2n, k] for the silu-mul epilogue) share an element
    type; c is [m, n] in that type, or float32 (always for the residual epilogue,
    where the product is added into c in place).  bfloat16 operands go to the
    tensor cores, float32 operands to the CUDA cores (true 32-bit)."""
    if a.dtype == torch.bfloat16 and USE_TENSOR_CORES[0]:
        if err is None:
            err = _tc_err.get(a.device)
            if err is None:
                err = _tc_err[a.device] = new_error_word(a.device)
        if gemm_nt_tc(a, w, c, epilogue, err):
            return
    gemm_nt_simt(a, w, c, epilogue)


# ---------------------------------------------------------------------------
# library "seq": heads of unequal sizes, mixers with a carried state, routed experts
# ---------------------------------------------------------------------------

RULE_DELTA, RULE_WKV, RULE_GLA = 0, 1, 2


def qkv_finish(qkv, q_out, pages, q_gain, k_gain, cos, sin, positions, token_req, block_table, nq: int, nkv: int,
               d: int, dv: int, pad: int, rot_dim: int, eps: float, whole_projection: bool, has_kv: bool,
               write_cache: bool, err, bias=None, q_temp=None) -> None:
    """Finishes a projection ``qkv`` [tokens, nq*d (+ nkv*d + nkv*dv)]: RMSNorm of q and of k (over
    the whole projection, or per head), rotation of the first ``rot_dim`` elements of each head,
    queries to ``q_out`` [tokens, nq*pad] and keys and values into ``pages``
    [num_pages, 2, nkv, page_size, pad], padded with zeros (csrc/heads_wide.cu).  ``bias`` (one
    element per column of ``qkv``, or None) is added first; ``q_temp`` = (coef, every): the query at
    position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1)."""
    tokens = qkv.shape[0]
    cols = nq * d + (nkv * (d + dv) if has_kv else 0)
    if qkv.shape[1] != cols or q_out.shape != (tokens, nq * pad) or q_out.dtype != qkv.dtype:
        raise KernelError("qkv_finish: shapes do not agree")
    gains = [g for g in (q_gain, k_gain) if g is not None]
    if any(g.dtype != gains[0].dtype for g in gains):
        raise KernelError("qkv_finish: gains of two element types")
    want_q = nq * d if whole_projection else d
    want_k = nkv * d if whole_projection else d
    if (q_gain is not None and q_gain.numel() != want_q) or (k_gain is not None and k_gain.numel() != want_k):
        raise KernelError("qkv_finish: gains do not match the projection")
    if write_cache:
        if pages.dtype != qkv.dtype or pages.shape[1:3] != (2, nkv) or pages.shape[4] != pad:
            raise KernelError("qkv_finish: cache pages do not match the projections")
        num_pages, page_size = pages.shape[0], pages.shape[3]
    else:
        num_pages, page_size = 0, 1
    if rot_dim and (cos.shape != sin.shape or cos.shape[1] != rot_dim // 2):
        raise KernelError("qkv_finish: rotary tables do not match rot_dim")
    if bias is not None and bias.numel() != cols:
        raise KernelError("qkv_finish: the bias does not match the projection")
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 1)
    _check(library("seq").ls_qkv_finish(
        _dev(qkv, "qkv"), qkv.shape[1], _dev(q_out, "q_out"), _opt(pages if write_cache else None, "pages"),
        _code(qkv), _opt(q_gain, "q_gain"), _opt(k_gain, "k_gain"), _code(gains[0]) if gains else F32,
        _opt(cos if rot_dim else None, "cos", torch.float32), _opt(sin if rot_dim else None, "sin", torch.float32),
        _dev(positions, "positions", torch.int32), _dev(token_req, "token_req", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[-1], tokens, nq, nkv, d, dv, pad, rot_dim,
        page_size, num_pages, cos.shape[0] if rot_dim else 0, float(eps), 2 if whole_projection else 1,
        1 if has_kv else 0, 1 if write_cache else 0, _opt(bias, "bias"), _code(bias) if bias is not None else F32,
        coef, every, _dev(err, "err", torch.int32), _stream()), "qkv_finish")


def latent_finish(proj, q_out, pages, gain, cos, sin, positions, token_req, block_table, heads: int, d: int, dr: int,
                  rank: int, pad: int, eps: float, interleaved: bool, write_cache: bool, err, w_fold=None,
                  kv=None) -> None:
    """Between the projections and the attention over a cached latent (csrc/latent.cu).  ``proj`` [tokens, >=
    heads (d + dr)]: every head's plain and rotated query part; ``kv`` [tokens, >= rank + dr]: the latent and the
    shared rotated key part (default: the columns of ``proj`` behind the queries; unused when no cache is
    written).  Writes the rotated query parts (and the padding) to columns rank .. pad of every head of
    ``q_out`` [tokens, heads pad], and [norm(latent) ; rotated key part ; 0] / [norm(latent) ; 0] as the token's
    key and value rows into ``pages`` [num_pages, 2, 1, page_size, pad].  With ``w_fold`` [heads, rank, d] it also
    writes columns 0 .. rank of every head, plain query part @ w_fold[head].T, with the bits of ``heads_product`` (for
    steps of few tokens: every token's block reads all of ``w_fold``)."""
    tokens = proj.shape[0]
    if w_fold is not None and (tuple(w_fold.shape) != (heads, rank, d) or w_fold.dtype != proj.dtype):
        raise KernelError("latent_finish: the fold's weights do not match")
    if q_out.shape != (tokens, heads * pad) or q_out.dtype != proj.dtype:
        raise KernelError("latent_finish: shapes do not agree")
    if write_cache:
        if kv is None:
            kv = proj[:, heads * (d + dr):]
        if kv.shape[0] != tokens or kv.shape[1] < rank + dr or kv.dtype != proj.dtype or gain.numel() != rank:
            raise KernelError("latent_finish: the latent's columns do not match")
    kp, kv_ld = _rows(kv, "kv") if write_cache else (0, 0)
    if write_cache and (pages.dtype != proj.dtype or tuple(pages.shape[1:3]) != (2, 1) or pages.shape[4] != pad):
        raise KernelError("latent_finish: cache pages do not match")
    if dr and (cos.shape != sin.shape or cos.shape[1] != dr // 2):
        raise KernelError("latent_finish: rotary tables do not match the rotated part")
    pp, ld = _rows(proj, "proj")
    _check(library("seq").ls_latent_finish(
        pp, ld, kp, kv_ld, _code(proj), _dev(q_out, "q_out"), _opt(pages if write_cache else None, "pages"),
        _opt(gain if write_cache else None, "gain"), _code(gain) if write_cache else F32, _opt(cos if dr else None, "cos", torch.float32), _opt(sin if dr else None, "sin", torch.float32),
        _dev(positions, "positions", torch.int32), _dev(token_req, "token_req", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[-1], tokens, heads, d, dr, rank, pad,
        pages.shape[3] if write_cache else 1, pages.shape[0] if write_cache else 0, cos.shape[0] if dr else 0,
        1 if interleaved else 0, 1 if write_cache else 0, float(eps), _opt(w_fold, "w_fold"),
        _dev(err, "err", torch.int32), _stream()), "latent_finish")


def heads_product(a, a_head_stride: int, w, out, out_head_stride: int) -> None:
    """out[t, h out_head_stride + n] = sum_k a[t, h a_head_stride + k] w[h, n, k] for every head h at once:
    ``a`` and ``out`` are [tokens, columns] (views of some columns of wider tensors are fine), ``w`` [heads, n, k]."""
    heads, n, k = w.shape
    ap, a_ld = _rows(a, "a")
    op, o_ld = _rows(out, "out")
    if a.shape[0] != out.shape[0] or a.dtype != w.dtype or out.dtype != w.dtype:
        raise KernelError("heads_product: shapes or types do not agree")
    if (heads - 1) * a_head_stride + k > a.shape[1] or (heads - 1) * out_head_stride + n > out.shape[1]:
        raise KernelError("heads_product: the heads do not fit the rows")
    _check(library("seq").ls_heads_product(ap, a_ld, a_head_stride, _dev(w, "w"), op, o_ld, out_head_stride, _code(w),
                                           a.shape[0], heads, n, k, _stream()), "heads_product")


def sigmoid_power_decay(z, bias, tau: float) -> None:
    """z <- sigmoid(z + bias)^(1 / tau) in place (float32 [tokens, channels]), through its logarithm."""
    _check(library("seq").ls_sigmoid_power_decay(_dev(z, "z", torch.float32), _dev(bias, "bias", torch.float32),
                                                 z.numel(), z.shape[1], float(tau), _stream()), "sigmoid_power_decay")


def find_portions(token_slot, out, cap: int, err) -> None:
    """out int32 [1 + 3 cap]: the number of portions of the step's token axis, then (first token,
    tokens, slot) of each, from ``token_slot`` alone (csrc/recurrent.cu)."""
    if out.numel() < 1 + 3 * cap:
        raise KernelError("find_portions: the list is too short")
    _check(library("seq").ls_find_portions(_dev(token_slot, "token_slot", torch.int32), token_slot.numel(),
                                           _dev(out, "out", torch.int32), cap, _dev(err, "err", torch.int32),
                                           _stream()), "find_portions")


def delta_prep(proj, conv_w, dt_bias, a_log, state, token_slot, qkv, decay, beta, heads: int, groups: int, dk: int,
               dv: int, taps: int, unit_eps: float) -> None:
    """What lies between the projections and the gated delta rule, a token a block: causal
    convolution (carried inputs from ``state``) and silu of q, k, v, unit q and k (q scaled),
    beta = sigmoid of its column, and the decay per key channel, made in place from the output
    of its low-rank map: ``decay`` <- exp(-exp(a_log[head]) softplus(decay + dt_bias)).  float32 out.
    ``proj`` [tokens, >= 2 G dk + H dv + H]."""
    f32 = torch.float32
    _check(library("seq").ls_delta_prep(
        _dev(proj, "proj"), proj.shape[1], _code(proj), _dev(conv_w, "conv_w", f32), _dev(dt_bias, "dt_bias", f32),
        _dev(a_log, "a_log", f32), _dev(state, "state", f32), state.shape[1],
        _dev(token_slot, "token_slot", torch.int32), _dev(qkv, "qkv", f32), _dev(decay, "decay", f32),
        _dev(beta, "beta", f32), proj.shape[0], heads, groups, dk, dv, taps, float(unit_eps), _stream()), "delta_prep")


def double_exp_decay(z, bias) -> None:
    """z <- exp(-exp(z + bias)) in place (float32 [tokens, channels]): a decay from the output of
    its low-rank map."""
    _check(library("seq").ls_double_exp_decay(_dev(z, "z", torch.float32), _dev(bias, "bias", torch.float32),
                                              z.numel(), z.shape[1], _stream()), "double_exp_decay")


def shift_mix(x, mu, state, prev_offset: int, token_slot, out) -> None:
    """out[s, t] = x[t] + (x[t - 1] - x[t]) * mu[s], the token before a portion's first one taken
    from ``state[slot, prev_offset:]``."""
    tokens, width = x.shape
    if out.shape != (mu.shape[0], tokens, width) or out.dtype != x.dtype:
        raise KernelError("shift_mix: shapes do not agree")
    _check(library("seq").ls_shift_mix(
        _dev(x, "x"), _code(x), _dev(mu, "mu", torch.float32), _dev(state, "state", torch.float32), state.shape[1],
        prev_offset, _dev(token_slot, "token_slot", torch.int32), _dev(out, "out"), tokens, width, mu.shape[0],
        _stream()), "shift_mix")


def tanh_rows(x) -> None:
    """x <- tanh(x) in place."""
    _check(library("seq").ls_tanh_rows(_dev(x, "x"), _code(x), x.numel(), _stream()), "tanh_rows")


def state_rule(rule: int, dtype, portions, max_portions: int, state, in_a, in_b, in_v, decay, beta, bonus, out,
               carry_src, carry_width: int, carry_rows: int, heads: int, groups: int, dk: int, dv: int,
               out_scale: float = 1.0, decay_fixed: bool = False) -> None:
    """(``decay_fixed``: ``decay`` is one row [heads dk] that serves every token.)  Walks every portion of the step through a state rule (RULE_DELTA, RULE_WKV, RULE_GLA), reading and
    writing ``state[slot]`` (float32: the matrix state, then the carried inputs).  RULE_GLA (S <- diag(decay) S
    + k v^T, o = out_scale S^T q) carries nothing else; its ``in_a``, ``in_b``, ``in_v`` (q, k, v in the engine's
    type) may be views of columns of one wider tensor."""
    in_ld = 0
    if rule == RULE_GLA:
        (pa, in_ld), (pb, ldb), (pv, ldv) = _rows(in_a, "in_a"), _rows(in_b, "in_b"), _rows(in_v, "in_v")
        if not (in_ld == ldb == ldv) or not (in_a.dtype == in_b.dtype == in_v.dtype == dtype):
            raise KernelError("state_rule: q, k and v must be columns of rows of one pitch, in the engine's type")
    else:
        pa, pb, pv = _dev(in_a, "in_a"), _opt(in_b, "in_b"), _opt(in_v, "in_v")
    _check(library("seq").ls_state_rule(
        rule, _DTYPE_CODE[dtype], _dev(portions, "portions", torch.int32), max_portions,
        _dev(state, "state", torch.float32), state.shape[1], pa, pb, pv,
        _dev(decay, "decay", torch.float32), _opt(beta, "beta", torch.float32), _opt(bonus, "bonus", torch.float32),
        _dev(out, "out", torch.float32), _opt(carry_src, "carry_src", dtype),
        carry_src.shape[1] if carry_src is not None else 0, carry_width,
        carry_rows, heads, groups, dk, dv, in_ld, float(out_scale), 0 if decay_fixed else -1, _stream()), "state_rule")


def head_rms_gate(o, gain, gate_f32, gate_x, out, heads: int, dv: int, gain_shared: bool, eps: float,
                  gate_logit: bool = False) -> None:
    """out = o / rms_per_head(o) * gain * gate, where the gate is ``gate_f32`` as it is (or its
    sigmoid, ``gate_logit``), or silu(``gate_x``); ``gate_x`` may be a view of some columns of a
    wider tensor."""
    gate_p, gate_ld = (0, 0)
    if gate_x is not None:
        if gate_x.dtype != out.dtype or gate_x.shape != (o.shape[0], heads * dv):
            raise KernelError("head_rms_gate: the gate does not match the read-out")
        gate_p, gate_ld = _rows(gate_x, "gate_x")
    _check(library("seq").ls_head_rms_gate(
        _dev(o, "o", torch.float32), _dev(gain, "gain", torch.float32), _opt(gate_f32, "gate_f32", torch.float32),
        gate_p, _dev(out, "out"), _code(out), o.shape[0], heads, dv,
        1 if gain_shared else 0, 1 if gate_logit else 0, float(eps), gate_ld, _stream()), "head_rms_gate")


def unit_gates(proj, x_at: int, x_bias, conv_w, conv_b, state, token_slot, w_r, w_i, b_r, b_i, rate, a_out, b_out,
               blocks: int, taps: int, c: float) -> None:
    """Decays and input terms of a gated recurrent unit per channel (csrc/unit_recurrence.cu): ``proj`` [tokens, *]
    holds the unit's x projection from column ``x_at`` on; ``w_r``, ``w_i`` [blocks, in, out] in the type of ``proj``."""
    tokens, width = a_out.shape
    bw = width // blocks
    if tuple(w_r.shape) != (blocks, bw, bw) or tuple(w_i.shape) != (blocks, bw, bw) or w_r.dtype != proj.dtype \
            or b_out.shape != a_out.shape or conv_w.shape != (width, taps) or state.shape[1] < taps * width:
        raise KernelError("unit_gates: shapes do not agree")
    pp, ld = _rows(proj, "proj")
    _check(library("seq").ls_unit_gates(
        pp, ld, int(x_at), _code(proj), _dev(x_bias, "x_bias", torch.float32), _dev(conv_w, "conv_w", torch.float32),
        _dev(conv_b, "conv_b", torch.float32), _dev(state, "state", torch.float32), state.stride(0),
        _dev(token_slot, "token_slot", torch.int32), _dev(w_r, "w_r"), _dev(w_i, "w_i"), _dev(b_r, "b_r", torch.float32),
        _dev(b_i, "b_i", torch.float32), _dev(rate, "rate", torch.float32), _dev(a_out, "a_out", torch.float32),
        _dev(b_out, "b_out", torch.float32), tokens, width, int(blocks), int(taps), float(c), _stream()), "unit_gates")


def unit_scan(portions, max_portions: int, a, b, proj, y_at: int, x_at: int, y_bias, x_bias, state, out, taps: int) -> None:
    """S <- a S + b along every portion, out = S gelu(y + bias); the slot keeps S and the convolution's last
    ``taps`` - 1 inputs (csrc/unit_recurrence.cu)."""
    tokens, width = a.shape
    if out.shape != a.shape or out.dtype != proj.dtype or b.shape != a.shape:
        raise KernelError("unit_scan: shapes do not agree")
    pp, ld = _rows(proj, "proj")
    _check(library("seq").ls_unit_scan(
        _dev(portions, "portions", torch.int32), int(max_portions), _dev(a, "a", torch.float32), _dev(b, "b", torch.float32),
        pp, ld, int(y_at), int(x_at), _code(proj), _dev(y_bias, "y_bias", torch.float32), _dev(x_bias, "x_bias", torch.float32),
        _dev(state, "state", torch.float32), state.stride(0), _dev(out, "out"), width, int(taps), _stream()), "unit_scan")


def rotate_rows(proj, q_at: int, k_at: int, v_at: int, cos, sin, positions, out, heads: int, dk: int, dv: int, rot_dim: int,
                k_scale: float, err) -> None:
    """out [tokens, 2 heads dk + heads dv] float32: the queries and keys of ``proj`` (columns from ``q_at`` / ``k_at``)
    with the first ``rot_dim`` elements of every head rotated (halves layout), the keys times ``k_scale``, then the values."""
    tokens = out.shape[0]
    if out.shape[1] != heads * (2 * dk + dv) or proj.shape[0] != tokens:
        raise KernelError("rotate_rows: shapes do not agree")
    if rot_dim and (cos.shape != sin.shape or cos.shape[1] != rot_dim // 2):
        raise KernelError("rotate_rows: rotary tables do not match rot_dim")
    pp, ld = _rows(proj, "proj")
    _check(library("seq").ls_rotate_rows(
        pp, ld, int(q_at), int(k_at), int(v_at), _code(proj), _opt(cos if rot_dim else None, "cos", torch.float32),
        _opt(sin if rot_dim else None, "sin", torch.float32), _dev(positions, "positions", torch.int32),
        _dev(out, "out", torch.float32), tokens, heads, dk, dv, rot_dim, cos.shape[0] if rot_dim else 0, float(k_scale),
        _dev(err, "err", torch.int32), _stream()), "rotate_rows")


def experts_tile_rows(tensor_cores: bool = False) -> int:
    """The most rows of a tile of the experts' products: of the CUDA-core product, or of the
    tensor-core one."""
    lib = library("seq")
    return int(lib.ls_experts_tc_tile_rows() if tensor_cores else lib.ls_experts_tile_rows())


def experts_route(logits, top: int, ids, weights, experts: int | None = None, softmax: bool = False,
                  correction=None) -> None:
    """The ``top`` experts of every token and their weights, from float32 ``logits`` [tokens, >= experts] (the
    first ``experts`` columns; default all; a view of some columns of a wider tensor is fine).  The weight is the sigmoid of the logit, or with ``softmax`` the
    softmax over the experts; ``correction`` (float32 [experts]) is added to it for the choice alone."""
    tokens = logits.shape[0]
    experts = logits.shape[1] if experts is None else int(experts)
    if correction is not None and correction.numel() != experts:
        raise KernelError("experts_route: the correction does not match the experts")
    if logits.dtype != torch.float32:
        raise KernelError("experts_route: logits must be float32")
    lp, l_ld = _rows(logits, "logits")
    _check(library("seq").ls_experts_route(lp, l_ld, tokens, experts, top,
                                           int(softmax), _opt(correction, "correction", torch.float32),
                                           _dev(ids, "ids", torch.int32), _dev(weights, "weights", torch.float32),
                                           _stream()), "experts_route")


def experts_mix(y, pair_row, ids, weights, real: int, x, out, shared=None, shared_gate=None, store: bool = False) -> None:
    """out[t] (+)= sum_r weights[t, r] * (y[pair_row[t, r]] if ids[t, r] < real else x[t]) + sigmoid(shared_gate[t])
    * shared[t], in order of rank: ids from ``real`` on are identity experts; ``weights`` None counts as one,
    ``shared`` (float32 [tokens, width]) None as absent, ``shared_gate`` (a float32 column, one logit per token) None
    as a weight of one.  ``store``: ``out`` is written instead of added to."""
    tokens, width = out.shape
    top = ids.shape[1]
    if x.shape != (tokens, width) or (shared is not None and tuple(shared.shape) != (tokens, width)):
        raise KernelError("experts_mix: shapes do not agree")
    gate_ld = 0
    if shared_gate is not None:
        if shared_gate.dtype != torch.float32 or shared_gate.shape[0] != tokens or not shared_gate.is_cuda:
            raise KernelError("experts_mix: the shared expert's gate does not match")
        gate_ld = shared_gate.stride(0) if tokens > 1 else 1
    _check(library("seq").ls_experts_mix(
        _opt(y, "y", torch.float32), _dev(pair_row, "pair_row", torch.int32), _dev(ids, "ids", torch.int32),
        _opt(weights, "weights", torch.float32), int(real), _dev(x, "x"), _code(x), _opt(shared, "shared", torch.float32),
        shared_gate.data_ptr() if shared_gate is not None else 0, gate_ld, _dev(out, "out", torch.float32), tokens, top,
        width, 1 if store else 0, _stream()), "experts_mix")


def experts_plan(ids, weights, experts: int, tile_rows: int, plan, max_tiles: int, row_token, row_weight, pair_row,
                 err) -> None:
    tokens, top = ids.shape
    _check(library("seq").ls_experts_plan(
        _dev(ids, "ids", torch.int32), _dev(weights, "weights", torch.float32), tokens, top, experts, tile_rows,
        _dev(plan, "plan", torch.int32), max_tiles, _dev(row_token, "row_token", torch.int32),
        _dev(row_weight, "row_weight", torch.float32), _dev(pair_row, "pair_row", torch.int32),
        _dev(err, "err", torch.int32), _stream()), "experts_plan")


def experts_route_plan(logits, top: int, ids, weights, experts: int, softmax: bool, correction, real: int, tile_rows: int,
                       plan, max_tiles: int, row_token, row_weight, pair_row, err) -> None:
    """``experts_route`` and ``experts_plan`` (over the first ``real`` experts) in one launch of one block, for steps
    of few tokens: the same choices, weights and plan."""
    tokens = logits.shape[0]
    if logits.dtype != torch.float32 or (correction is not None and correction.numel() != experts):
        raise KernelError("experts_route_plan: the logits or the correction do not match")
    lp, l_ld = _rows(logits, "logits")
    _check(library("seq").ls_experts_route_plan(
        lp, l_ld, tokens, experts, top, int(softmax), _opt(correction, "correction", torch.float32),
        _dev(ids, "ids", torch.int32), _dev(weights, "weights", torch.float32), real, tile_rows,
        _dev(plan, "plan", torch.int32), max_tiles, _dev(row_token, "row_token", torch.int32),
        _dev(row_weight, "row_weight", torch.float32), _dev(pair_row, "pair_row", torch.int32),
        _dev(err, "err", torch.int32), _stream()), "experts_route_plan")


def experts_product(mode: int, plan, max_tiles: int, a, row_token, row_weight, w, c) -> None:
    """mode 0: c[row] = relu((a[row_token[row]] * row_weight[row]) @ w[e].T)^2; mode 1: c[row] = a[row] @ w[e].T
    in float32; mode 2: c[row_token[row]] += a[row] @ w[e].T (float32; for a token's one expert); mode 3:
    c[row] = (a[row_token[row]] * row_weight[row]) @ w[e].T in float32 (``row_weight`` None: one); rows sorted by
    expert as ``plan`` says.  w [experts, n, k]."""
    n, k = w.shape[1], w.shape[2]
    if a.shape[1] != k or c.shape[1] != n or a.dtype != w.dtype:
        raise KernelError("experts_product: shapes do not agree")
    _check(library("seq").ls_experts_product(
        mode, _code(a), _dev(plan, "plan", torch.int32), max_tiles, _dev(a, "a"),
        _dev(row_token, "row_token", torch.int32), _opt(row_weight, "row_weight", torch.float32), _dev(w, "w"),
        _dev(c, "c"), n, k, _stream()), "experts_product")


def experts_combine(y, pair_row, residual, top: int) -> None:
    tokens, width = residual.shape
    _check(library("seq").ls_experts_combine(_dev(y, "y", torch.float32), _dev(pair_row, "pair_row", torch.int32),
                                             _dev(residual, "residual", torch.float32), tokens, top, width, _stream()),
           "experts_combine")


def experts_gather(x, row_token, row_weight, out) -> None:
    """out[row] = x[row_token[row]] * row_weight[row] (bfloat16; ``row_weight`` None: a copy): the sorted,
    scaled rows that the tensor-core product of the experts' first matrices reads."""
    rows, width = out.shape
    if x.shape[1] != width or x.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("experts_gather: shapes or types do not agree")
    _check(library("seq").ls_experts_gather(_dev(x, "x"), _dev(row_token, "row_token", torch.int32),
                                            _opt(row_weight, "row_weight", torch.float32), _dev(out, "out"), rows,
                                            width, _stream()), "experts_gather")


def experts_product_tc(mode: int, plan, max_tiles: int, a, w, c, err, row_token=None) -> bool:
    """The experts' product on tcgen05 (csrc/experts_tc.cu): a [rows, k] bfloat16 sorted by expert, w
    [experts, n, k] bfloat16; mode 0: c = relu(a @ w[e].T)^2 (bfloat16), mode 1: c = a @ w[e].T (float32),
    mode 2: c[row_token[row]] += a[row] @ w[e].T (float32 [tokens, n]; for a token's one expert).
    Returns False, having launched nothing, for what TMA cannot address."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not USE_TENSOR_CORES[0]:
        return False
    n, k = w.shape[1], w.shape[2]
    if a.shape[1] != k or c.shape[1] != n or (mode != 2 and c.shape[0] != a.shape[0]) \
            or c.dtype != (torch.bfloat16 if mode == 0 else torch.float32) or (mode == 2 and row_token is None):
        raise KernelError("experts_product_tc: shapes or types do not agree")
    status = library("seq").ls_experts_product_tc(
        mode, _dev(plan, "plan", torch.int32), max_tiles, _dev(a, "a"), a.shape[0], _dev(w, "w"), w.shape[0],
        _opt(row_token, "row_token", torch.int32), _dev(c, "c"), n, k, _dev(err, "err", torch.int32), _stream())
    if status in (-2, -3):
        return False
    _check(status, "experts_product_tc")
    return True
