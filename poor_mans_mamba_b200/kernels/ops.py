"""Python face of the CUDA kernels: argument checks, then one C call per op on the
current CUDA stream.  Nothing here computes on the host and nothing falls back: a tensor
that is not on a CUDA device, a size a kernel cannot take, or a missing library raises.

Matrix products go to the library (cuBLAS through ``torch.mm``), as the reference sends
its linear layers to ``cublasSgemm`` (src/ops/gpu/linear.cu:3-21); in float32 the
reduced-precision matrix mode is switched off for the call.
"""
from __future__ import annotations

import ctypes
import os
import weakref
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import build as _build

Tensor = torch.Tensor

PMM_ERR_BAD_ARGUMENT = 1001


class KernelError(RuntimeError):
    """A kernel launch was refused or failed."""


_SIGNATURES = {
    "pmm_embed": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p],
    "pmm_add_postnorm_rmsnorm": [c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_float, c_void_p, c_float,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "pmm_add_rmsnorm": [c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_float, c_void_p,
                        c_void_p, c_int, c_int, c_int, c_void_p],
    "pmm_scale_f32": [c_void_p, c_float, c_longlong, c_void_p],
    "pmm_cast_scale": [c_void_p, c_void_p, c_float, c_longlong, c_int, c_void_p],
    "pmm_conv1d_fwd": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_conv1d_window_update": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_conv1d_decode": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_ssm_scan_seq": [c_void_p, c_int, c_void_p, c_longlong, c_float, c_void_p, c_void_p,
                         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                         c_int, c_void_p, c_longlong, c_float, c_void_p, c_int, c_int, c_void_p],
    "pmm_ssd_supported": [c_int, c_int],
    "pmm_ssd_chunked": [c_void_p, c_int, c_void_p, c_longlong, c_float, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                        c_int, c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_float, c_void_p, c_void_p],
    "pmm_ssd_tc_supported": [c_int, c_int],
    "pmm_ssd_tc": [c_void_p, c_int, c_void_p, c_longlong, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                   c_longlong, c_float, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "pmm_gated_norm": [c_void_p, c_void_p, c_longlong, c_float, c_void_p, c_void_p, c_float, c_int,
                       c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_qkv_rope_store": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_float,
                           c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                           c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                           c_void_p],
    "pmm_kv_store": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                     c_int, c_int, c_void_p],
    "pmm_paged_attention": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "pmm_kept_first_merge": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_hc_mix_norm": [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_normed_sum": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_int, c_int, c_int, c_int,
                       c_void_p],
    "pmm_rope_pairs_store": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p],
    "pmm_delta_scan": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong,
                       c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                       c_int, c_int, c_int, c_float, c_float, c_int, c_void_p],
    "pmm_recurrent_chunked_supported": [c_int, c_int],
    "pmm_recurrent_chunked_scratch": [c_int, c_int, c_int],
    "pmm_recurrent_chunked": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong,
                              c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p],
    "pmm_decay_scan": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_flash_supported": [c_int, c_int, c_int],
    "pmm_flash_paged_attention": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "pmm_l2_prefetch": [c_void_p, c_void_p, c_int, c_void_p],
    "pmm_attention_tc_supported": [c_int, c_int, c_int, c_int],
    "pmm_attention_tc": [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                         c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                         c_void_p, c_void_p, c_void_p, c_void_p],
    "pmm_skinny_chain": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "pmm_flash_decode_attention": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_float,
                                   c_float, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "pmm_decode_attention_tma_supported": [c_int, c_int, c_int, c_int],
    "pmm_decode_attention_tma": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_float, c_float,
                                 c_float, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_void_p],
    "pmm_flash_combine": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_skinny_gemm": [c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_int,
                        c_float, c_void_p, c_longlong, c_void_p, c_int, c_float, c_void_p, c_longlong, c_void_p,
                        c_int, c_void_p],
    "pmm_skinny_gemm_f32out": [c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_float, c_void_p, c_longlong,
                               c_void_p],
    "pmm_skinny_tc_supported": [c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong],
    "pmm_skinny_tc": [c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_float, c_void_p, c_longlong,
                      c_void_p, c_int, c_float, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p],
    "pmm_tc_gemm_supported": [c_int, c_int, c_int, c_longlong, c_longlong],
    "pmm_tc_gemm": [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_float,
                    c_void_p, c_void_p],
    "pmm_tc_gemm_act": [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_float,
                        c_float, c_float, c_void_p, c_void_p],
    "pmm_silu_mul": [c_void_p, c_longlong, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "pmm_gelu_tanh_mul": [c_void_p, c_longlong, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "pmm_add_row_bias": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "pmm_add_tanh_norm": [c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "pmm_sigmoid_gate": [c_void_p, c_longlong, c_void_p, c_longlong, c_float, c_void_p, c_longlong, c_int, c_int, c_int,
                         c_int, c_int, c_void_p],
    "pmm_clamped_glu": [c_void_p, c_longlong, c_float, c_float, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "pmm_moe_route": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                      c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p],
    "pmm_moe_plan": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "pmm_moe_tile_rows": [c_int],
    "pmm_moe_gemm": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                     c_int, c_float, c_float, c_float, c_void_p, c_int, c_int, c_void_p],
    "pmm_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_moe_tc_tile_rows": [],
    "pmm_moe_tc_supported": [c_int, c_int, c_longlong],
    "pmm_moe_gather_rows": [c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p],
    "pmm_moe_tc_gemm": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                        c_float, c_float, c_float, c_void_p, c_void_p, c_void_p],
    "pmm_latent_norm_store": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p],
    "pmm_latent_query_rot": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_void_p],
    "pmm_head_gate": [c_void_p, c_longlong, c_void_p, c_longlong, c_float, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                      c_void_p],
    "pmm_token_gated_update_fits": [c_int, c_int],
    "pmm_token_gated_update": [c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_void_p, c_longlong, c_int,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_cast_rows": [c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p],
    "pmm_relu_squared": [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p],
    "pmm_sample_rows": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                        c_void_p, c_void_p, c_void_p],
}

_FUNCS = {}
launch_count = 0  # kernels of this library launched since import (library GEMMs not counted)


def _fn(name: str):
    f = _FUNCS.get(name)
    if f is None:
        lib = _build.load()
        try:
            f = getattr(lib, name)
        except AttributeError as exc:
            raise KernelError(f"kernel library has no symbol {name}; rebuild it") from exc
        f.argtypes = _SIGNATURES[name]
        f.restype = c_int
        _FUNCS[name] = f
    return f


def _call(name: str, *args) -> None:
    global launch_count
    rc = _fn(name)(*args)
    launch_count += 1
    if rc != 0:
        if rc == PMM_ERR_BAD_ARGUMENT:
            raise KernelError(f"{name}: sizes or arguments outside what the kernel supports")
        raise KernelError(f"{name}: CUDA error {rc} at launch")


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch: the raw getter takes 0.3 us where
    building a torch.cuda.Stream object takes 3 to 15."""
    if _RAW_STREAM is not None:
        return _RAW_STREAM(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"storage type must be float32 or bfloat16, got {t.dtype}")


def _ptr(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()



# ----------------------------------------------------------------------------- status of bounded waits
class _StatusWatch:
    """The status words of one device and their host copy.

    Kernels whose threads wait on one another (mbarrier waits of the tcgen05 kernels, the grid
    barrier of skinny_chain) bound every wait; a wait that gives up writes a code into a status
    word, the block abandons its tile and returns, and the output of that launch is incomplete.
    ``words[0]`` is shared by the tensor-core kernels, ``words[1]`` by the chain.  The engine
    copies the words to pinned memory with the results it fetches anyway (`snapshot`) and looks
    at the copy once the host has waited for that fetch (`check`)."""

    def __init__(self, device: torch.device):
        self.device = device
        self.words = torch.zeros(2, dtype=torch.int32, device=device)
        self.host = torch.zeros(2, dtype=torch.int32, pin_memory=True)
        self.counters: "weakref.WeakSet" = weakref.WeakSet()

    def snapshot(self) -> None:
        self.host.copy_(self.words, non_blocking=True)

    def check(self) -> None:
        tc, chain = int(self.host[0]), int(self.host[1])
        if tc == 0 and chain == 0:
            return
        # leave the device usable: clear the words and whatever a half-finished launch left behind
        self.words.zero_()
        self.host.zero_()
        for c in list(self.counters):
            c.zero_()
        raise KernelError(f"a bounded wait inside a kernel gave up on {self.device} (tensor-core kernels: code {tc}; "
                          f"grid-barrier chain: code {chain}): the step's results are incomplete and were discarded")


_WATCHES: Dict[torch.device, _StatusWatch] = {}


def _watch(device: torch.device) -> _StatusWatch:
    device = torch.device(device)
    if device.index is None and device.type == "cuda":
        device = torch.device("cuda", torch.cuda.current_device())
    w = _WATCHES.get(device)
    if w is None:
        w = _StatusWatch(device)
        _WATCHES[device] = w
    return w


def watch_split_counter(counter: Tensor) -> None:
    """Registers an attention split counter (zero between launches) to be cleared when a launch
    was abandoned half-way."""
    _watch(counter.device).counters.add(counter)


def status_snapshot(device) -> None:
    """Enqueue the copy of the device's status words to pinned memory on the current stream."""
    _watch(device).snapshot()


def check_status(device, wait: bool = False) -> None:
    """Raise KernelError if the last snapshot that has reached the host shows an abandoned wait.
    ``wait``: take a snapshot now and wait for the current stream first."""
    w = _watch(device)
    if wait:
        w.snapshot()
        torch.cuda.current_stream(w.device).synchronize()
    w.check()


def _cuda(*tensors: Optional[Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only (no CPU path exists)")


def _rows_view(t: Tensor, what: str) -> int:
    """Row stride (elements) of a 2-D view whose rows are contiguous."""
    if not (t.dim() == 2 and t.stride(1) == 1):
        raise KernelError(f"{what}: need a 2-D view with unit column stride")
    return t.stride(0)


def _f32vec(t: Optional[Tensor], n: int, what: str) -> None:
    if t is not None:
        if not (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n):
            raise KernelError(f"{what}: need a contiguous float32 vector of {n}")


def _i32(t: Tensor, what: str) -> None:
    if not (t.dtype == torch.int32 and t.is_contiguous()):
        raise KernelError(f"{what}: need contiguous int32")


# ----------------------------------------------------------------------------- library GEMM
def padded_rows(n_rows: int) -> int:
    """The row count a library product of ``n_rows`` rows is issued with.  The library chooses a
    kernel per (M, N, K) and the first call with a new M costs about 1.4 ms on the host (measured:
    18 us once the shape is known); a server sees a new token count in almost every step.  Rounded
    up to a multiple of 64 (128 from 1,024 rows, 256 from 4,096) the shapes recur.  The extra rows
    are scratch: the step's arena reserves them behind every matrix it hands out."""
    if n_rows <= 64:
        return n_rows
    step = 64 if n_rows < 1024 else (128 if n_rows < 4096 else 256)
    return (n_rows + step - 1) // step * step


def _with_rows(t: Tensor, rows: int) -> Optional[Tensor]:
    """``t`` [T, n] seen with ``rows`` >= T rows of the same stride, if its storage reaches that far."""
    if t.dim() != 2 or t.stride(1) != 1:
        return None
    last = t.storage_offset() + (rows - 1) * t.stride(0) + t.shape[1]
    if last * t.element_size() > t.untyped_storage().nbytes():
        return None
    return t.as_strided((rows, t.shape[1]), t.stride())


def _mm(x: Tensor, weight: Tensor, out: Tensor, **kw) -> None:
    """The library product; with `padded_rows(T)` rows where ``out`` is a whole matrix of the step's
    arena (which marks it with the rows it keeps behind it) and x's storage reaches as far.  What
    the extra rows of x hold does not matter, rows being independent, and nothing reads the extra
    rows of out."""
    n = x.shape[0]
    if n > 64:
        rows = padded_rows(n)
        if rows != n and getattr(out, "_scratch_rows", 0) >= rows:
            # matrices of the arena carry the padded view with them; a slice of one is widened here
            xp = x._with_scratch_rows if getattr(x, "_scratch_rows", 0) == rows else _with_rows(x, rows)
            op = out._with_scratch_rows if out._scratch_rows == rows else _with_rows(out, rows)
            if xp is not None and op is not None:
                x, out = xp, op
    torch.mm(x, weight.t(), out=out, **kw)


def linear(x: Tensor, weight: Tensor, out: Tensor) -> Tensor:
    """out[T, N] = x[T, K] @ weight[N, K]^T through the GEMM library."""
    _cuda(x, weight, out)
    if not (x.dtype == weight.dtype):
        raise KernelError(f"linear: activation {x.dtype} vs weight {weight.dtype}")
    if x.dtype == torch.float32:
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            _mm(x, weight, out)
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
    else:
        _mm(x, weight, out)
    return out


_MM_F32_OUT: Optional[bool] = None


def mm_has_f32_out() -> bool:
    """Whether the GEMM library gives a float32 result from bfloat16 operands directly."""
    global _MM_F32_OUT
    if _MM_F32_OUT is None:
        try:
            a = torch.zeros(8, 16, dtype=torch.bfloat16, device="cuda")
            torch.mm(a, a.t(), out_dtype=torch.float32)
            _MM_F32_OUT = True
        except (TypeError, RuntimeError):
            _MM_F32_OUT = False
    return _MM_F32_OUT


def linear_f32_out(x: Tensor, weight: Tensor, out: Tensor, scratch_low: Optional[Tensor], scale: float) -> None:
    """out (float32) = scale * (x @ weight^T) for bfloat16 operands.  The library is asked for
    a float32 result directly; a library build without that option gets a bfloat16 product
    that is widened (and scaled) by cast_scale."""
    _cuda(x, weight, out)
    if mm_has_f32_out():
        _mm(x, weight, out, out_dtype=torch.float32)
        if scale != 1.0:
            scale_f32_(out, scale)
    else:
        if not (scratch_low is not None):
            raise KernelError("linear_f32_out: needs a low-precision scratch buffer")
        torch.mm(x, weight.t(), out=scratch_low)
        cast_scale(out, scratch_low, scale)


# ----------------------------------------------------------------------------- own kernels
def embed(out: Tensor, table: Tensor, tokens: Tensor, mult: float, norm_weight: Optional[Tensor] = None,
          eps: float = 0.0) -> None:
    """out[t] = mult * table[tokens[t]] (float32); with ``norm_weight`` [D] the row is then divided by its root
    mean square (eps inside the root) and multiplied by the weight, all in float."""
    _cuda(out, table, tokens, norm_weight)
    T, D = out.shape
    if not (out.dtype == torch.float32 and out.is_contiguous()):
        raise KernelError("embed: out must be contiguous float32")
    if not (table.dim() == 2 and table.shape[1] == D and table.is_contiguous()):
        raise KernelError("embed: table must be [V, D]")
    _i32(tokens, "embed: tokens")
    if not (tokens.numel() == T):
        raise KernelError("embed: one token per output row")
    _f32vec(norm_weight, D, "embed: norm weight")
    _call("pmm_embed", out.data_ptr(), table.data_ptr(), tokens.data_ptr(), float(mult), T, D,
          table.shape[0], _dt(table), _ptr(norm_weight), float(eps), _stream())


def add_postnorm_rmsnorm(h: Optional[Tensor], branches: Sequence[Tuple[Tensor, float]], post_weight: Tensor, post_eps: float,
                         weight: Optional[Tensor], eps: float, out: Optional[Tensor], rows: Optional[Tensor] = None) -> None:
    """u = rmsnorm(s0*b0 + s1*b1) * post_weight;  h <- h + u (rows is None and h given);  out = rmsnorm(h + u) * weight
    (``weight`` None: out = h + u, or u alone without h).  With ``rows`` h is left as it is and out[r] comes from row
    rows[r].  One or two branches in the storage type; every statistic and sum is float."""
    _cuda(h, post_weight, weight, out, rows)
    if not (1 <= len(branches) <= 2):
        raise KernelError("add_postnorm_rmsnorm: one or two branches")
    T, D = branches[0][0].shape
    if h is not None and not (h.dtype == torch.float32 and h.shape == (T, D) and h.is_contiguous()):
        raise KernelError("add_postnorm_rmsnorm: the residual stream must be contiguous float32 [T, D]")
    if not (D * 4 <= 200 * 1024):
        raise KernelError(f"add_postnorm_rmsnorm: width {D} exceeds one block's shared memory")
    ptrs: List[Optional[int]] = [None, None]
    scales = [0.0, 0.0]
    dtype = _dt(branches[0][0])
    for i, (b, s) in enumerate(branches):
        _cuda(b)
        if not (b.shape == (T, D) and b.is_contiguous() and _dt(b) == dtype):
            raise KernelError("add_postnorm_rmsnorm: branches must be contiguous [T, D] of one storage type")
        ptrs[i], scales[i] = b.data_ptr(), float(s)
    _f32vec(post_weight, D, "add_postnorm_rmsnorm: post weight")
    _f32vec(weight, D, "add_postnorm_rmsnorm: weight")
    R = T
    if rows is not None:
        _i32(rows, "add_postnorm_rmsnorm: rows")
        R = rows.numel()
    if out is not None and not (out.shape == (R, D) and out.is_contiguous() and _dt(out) == dtype):
        raise KernelError("add_postnorm_rmsnorm: out must be contiguous [rows, D] of the branches' type")
    if out is None and (h is None or rows is not None):
        raise KernelError("add_postnorm_rmsnorm: nothing to write")
    _call("pmm_add_postnorm_rmsnorm", _ptr(h), ptrs[0], scales[0], ptrs[1], scales[1], post_weight.data_ptr(),
          float(post_eps), _ptr(weight), float(eps), _ptr(out), _ptr(rows), R, D, dtype, _stream())


def add_rmsnorm(h: Tensor, branches: Sequence[Tuple[Tensor, float]], weight: Optional[Tensor],
                eps: float, out: Optional[Tensor], rows: Optional[Tensor] = None) -> None:
    """h <- (h + s0*b0) + s1*b1 (rows is None), then out = rmsnorm(h) * weight.
    With ``rows`` (int32 row indices) h is left as it is and out[r] comes from row rows[r]."""
    _cuda(h, weight, out, rows)
    if not (h.dtype == torch.float32 and h.dim() == 2 and h.is_contiguous()):
        raise KernelError("add_rmsnorm: the residual stream must be contiguous float32 [T, D]")
    T, D = h.shape
    if not (len(branches) <= 2):
        raise KernelError("add_rmsnorm: at most two branches")
    if not (D * 4 <= 200 * 1024):
        raise KernelError(f"add_rmsnorm: width {D} exceeds one block's shared memory")
    ptrs: List[Optional[int]] = [None, None]
    scales = [0.0, 0.0]
    dtype = None
    for i, (b, s) in enumerate(branches):
        _cuda(b)
        if not (b.shape == h.shape and b.is_contiguous()):
            raise KernelError("add_rmsnorm: branch must be contiguous [T, D]")
        ptrs[i], scales[i] = b.data_ptr(), float(s)
        dtype = _dt(b) if dtype is None else dtype
        if not (_dt(b) == dtype):
            raise KernelError("add_rmsnorm: branches of different storage types")
    R = T
    if rows is not None:
        _i32(rows, "add_rmsnorm: rows")
        R = rows.numel()
    if out is not None:
        if not (weight is not None):
            raise KernelError("add_rmsnorm: a norm needs its weight")
        _f32vec(weight, D, "add_rmsnorm: weight")
        if not (out.shape == (R, D) and out.is_contiguous()):
            raise KernelError("add_rmsnorm: out must be contiguous [rows, D]")
        if not (dtype is None or _dt(out) == dtype):
            raise KernelError("add_rmsnorm: out and branches differ in storage type")
        dtype = _dt(out)
    if dtype is None:
        return  # nothing to add and nothing to write
    _call("pmm_add_rmsnorm", h.data_ptr(), ptrs[0], scales[0], ptrs[1], scales[1], _ptr(weight),
          float(eps), _ptr(out), _ptr(rows), R, D, dtype, _stream())


def add_tanh_norm(h: Optional[Tensor], branches: Sequence[Tuple[Tensor, float]],
                  post: Optional[Tuple[Tensor, Tensor, Tensor]], pre: Optional[Tuple[Tensor, Tensor, Tensor]],
                  out: Optional[Tensor], rows: Optional[Tensor] = None) -> None:
    """The norm y = tanh(alpha x) * w + b with the residual fold.  s = s0*b0 + s1*b1; with ``post``
    (alpha, w, b) s <- post(s); h <- h + s (rows is None); with ``pre`` (alpha, w, b) out = pre(h).
    h None: out = pre(s).  With ``rows`` h is left as it is and out[r] comes from row rows[r].
    alpha is a tensor of one float."""
    _cuda(h, out, rows)
    ref = h if h is not None else (branches[0][0] if branches else None)
    if ref is None or ref.dim() != 2:
        raise KernelError("add_tanh_norm: needs a stream or a branch [T, D]")
    T, D = ref.shape
    if h is not None and not (h.dtype == torch.float32 and h.is_contiguous()):
        raise KernelError("add_tanh_norm: the residual stream must be contiguous float32 [T, D]")
    if len(branches) > 2:
        raise KernelError("add_tanh_norm: at most two branches")
    ptrs: List[Optional[int]] = [None, None]
    scales = [0.0, 0.0]
    dtype = None
    for i, (b, s) in enumerate(branches):
        _cuda(b)
        if not (b.shape == (T, D) and b.is_contiguous()):
            raise KernelError("add_tanh_norm: branch must be contiguous [T, D]")
        ptrs[i], scales[i] = b.data_ptr(), float(s)
        dtype = _dt(b) if dtype is None else dtype
        if _dt(b) != dtype:
            raise KernelError("add_tanh_norm: branches of different storage types")
    trios = []
    for trio, what in ((post, "post"), (pre, "pre")):
        if trio is None:
            trios += [None, None, None]
            continue
        al, w, b = trio
        _cuda(al, w, b)
        _f32vec(w, D, f"add_tanh_norm: {what} weight")
        _f32vec(b, D, f"add_tanh_norm: {what} bias")
        if not (al.dtype == torch.float32 and al.numel() == 1):
            raise KernelError(f"add_tanh_norm: {what} alpha must be one float")
        trios += [al.data_ptr(), w.data_ptr(), b.data_ptr()]
    R = T
    if rows is not None:
        _i32(rows, "add_tanh_norm: rows")
        R = rows.numel()
    if out is not None:
        if pre is None:
            raise KernelError("add_tanh_norm: an output needs the norm's tensors")
        if not (out.shape == (R, D) and out.is_contiguous()):
            raise KernelError("add_tanh_norm: out must be contiguous [rows, D]")
        if not (dtype is None or _dt(out) == dtype):
            raise KernelError("add_tanh_norm: out and branches differ in storage type")
        dtype = _dt(out)
    if dtype is None:
        return
    _call("pmm_add_tanh_norm", _ptr(h), ptrs[0], scales[0], ptrs[1], scales[1], trios[0], trios[1], trios[2], trios[3],
          trios[4], trios[5], _ptr(out), _ptr(rows), R, D, dtype, _stream())


def scale_f32_(x: Tensor, s: float) -> None:
    _cuda(x)
    if not (x.dtype == torch.float32 and x.is_contiguous()):
        raise KernelError("scale_f32_: contiguous float32 only")
    _call("pmm_scale_f32", x.data_ptr(), float(s), x.numel(), _stream())


def cast_scale(out: Tensor, src: Tensor, s: float) -> None:
    _cuda(out, src)
    if not (out.dtype == torch.float32 and out.is_contiguous() and src.is_contiguous()
            and out.numel() == src.numel()):
        raise KernelError("cast_scale: contiguous tensors of equal size, float32 out")
    _call("pmm_cast_scale", out.data_ptr(), src.data_ptr(), float(s), src.numel(), _dt(src), _stream())


def _conv_common(x: Tensor, pre_scale: Tensor, pre_bias: Optional[Tensor], window: Tensor, K: int):
    C = x.shape[1]
    if K < 1:
        raise KernelError("conv1d: at least one tap")
    _f32vec(pre_scale, C, "conv1d: pre_scale")
    _f32vec(pre_bias, C, "conv1d: pre_bias")
    if not (window.dtype == torch.float32 and window.is_contiguous() and window.dim() == 3
            and tuple(window.shape[1:]) == (K - 1, C)):
        raise KernelError("conv1d: window must be float32 [slots, K-1, C]")
    return C


def conv1d_fwd(x: Tensor, pre_scale: Tensor, pre_bias: Optional[Tensor], weight: Tensor,
               bias: Optional[Tensor], window: Tensor, seq_of: Tensor, cu: Tensor, slots: Tensor,
               out: Tensor, weight_t: Optional[Tensor] = None, activation: bool = True) -> None:
    """Causal depthwise conv + SiLU (``activation`` False: the conv alone) over all tokens of the step; reads the windows.
    ``weight_t`` is the tap-major copy [K, C] of ``weight`` [C, K]; with it bfloat16 inputs take
    the vector kernel."""
    _cuda(x, pre_scale, pre_bias, weight, bias, window, seq_of, cu, slots, out, weight_t)
    ld = _rows_view(x, "conv1d: x")
    T = x.shape[0]
    if not (weight.dtype == torch.float32 and weight.dim() == 2 and weight.is_contiguous()
            and weight.shape[0] == x.shape[1]):
        raise KernelError("conv1d: weight must be contiguous float32 [C, K]")
    K = weight.shape[1]
    C = _conv_common(x, pre_scale, pre_bias, window, K)
    _f32vec(bias, C, "conv1d: bias")
    if not (out.shape == (T, C) and out.is_contiguous() and out.dtype == x.dtype):
        raise KernelError("conv1d: out must be [T, C]")
    if not (weight_t is None or (weight_t.dtype == torch.float32 and weight_t.is_contiguous()
            and weight_t.shape == (K, C))):
        raise KernelError("conv1d: weight_t must be contiguous float32 [K, C]")
    _call("pmm_conv1d_fwd", x.data_ptr(), ld, pre_scale.data_ptr(), _ptr(pre_bias), weight.data_ptr(),
          _ptr(weight_t), _ptr(bias), window.data_ptr(), seq_of.data_ptr(), cu.data_ptr(), slots.data_ptr(),
          out.data_ptr(), T, C, K, _dt(x), int(bool(activation)), _stream())


def conv1d_window_update(x: Tensor, pre_scale: Tensor, pre_bias: Optional[Tensor], window: Tensor,
                         cu: Tensor, slots: Tensor, n_seq: int, K: int) -> None:
    """Leaves the last K-1 conv inputs of every sequence in its window."""
    _cuda(x, pre_scale, pre_bias, window, cu, slots)
    ld = _rows_view(x, "conv1d: x")
    C = _conv_common(x, pre_scale, pre_bias, window, K)
    _call("pmm_conv1d_window_update", x.data_ptr(), ld, pre_scale.data_ptr(), _ptr(pre_bias),
          window.data_ptr(), cu.data_ptr(), slots.data_ptr(), n_seq, C, K, _dt(x), _stream())


def conv1d_decode(x: Tensor, pre_scale: Tensor, pre_bias: Optional[Tensor], weight: Tensor,
                  bias: Optional[Tensor], window: Tensor, slots: Tensor, out: Tensor,
                  activation: bool = True) -> None:
    """Conv + SiLU (``activation`` False: the conv alone) + window shift for a step in which every
    sequence brings one token."""
    _cuda(x, pre_scale, pre_bias, weight, bias, window, slots, out)
    ld = _rows_view(x, "conv1d: x")
    n_seq = x.shape[0]
    K = weight.shape[1]
    C = _conv_common(x, pre_scale, pre_bias, window, K)
    if not (weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape[0] == C):
        raise KernelError("conv1d: weight must be contiguous float32 [C, K]")
    _f32vec(bias, C, "conv1d: bias")
    if not (out.shape == (n_seq, C) and out.is_contiguous() and out.dtype == x.dtype):
        raise KernelError("conv1d: out must be [T, C]")
    _call("pmm_conv1d_decode", x.data_ptr(), ld, pre_scale.data_ptr(), _ptr(pre_bias),
          weight.data_ptr(), _ptr(bias), window.data_ptr(), slots.data_ptr(), out.data_ptr(), n_seq, C,
          K, _dt(x), int(bool(activation)), _stream())


def _gate_args(gate, out: Tensor, what: str):
    """(z pointer, row stride, scale, bias pointer) of an optional fused gate (z view, scale, bias)."""
    if gate is None:
        return None, 0, 0.0, None
    z, z_scale, z_bias = gate
    _cuda(z, z_bias)
    ld_z = _rows_view(z, f"{what}: z")
    if not (z.shape == out.shape and z.dtype == out.dtype):
        raise KernelError(f"{what}: z must match the output")
    _f32vec(z_bias, out.shape[1], f"{what}: z_bias")
    return z.data_ptr(), ld_z, float(z_scale), _ptr(z_bias)


def ssm_scan_seq(xbc: Tensor, dt_raw: Tensor, dt_scale: float, dt_shift: Tensor, a_log: Tensor,
                 d_skip: Tensor, state: Tensor, cu: Tensor, slots: Tensor, n_seq: int, out: Tensor,
                 n_groups: int, gate=None, one_token: bool = False, only_single: bool = False) -> None:
    """Token-serial Mamba2 recurrence from the saved state; state[slots, H, P, N] is updated.
    ``gate`` = (z view [T, I], z_scale, z_bias or None): the output is y * silu(z*z_scale + z_bias).
    ``one_token``: sequence s brings exactly token s (a decode step); ``cu`` is then not read.
    ``only_single``: only the sequences that bring exactly one token are walked (the lone tokens of
    a mixed step, whose longer portions the chunked scan takes); the others are left alone."""
    _cuda(xbc, dt_raw, dt_shift, a_log, d_skip, state, cu, slots, out)
    if not (state.dtype == torch.float32 and state.dim() == 4 and state.is_contiguous()):
        raise KernelError("ssm_scan: state must be contiguous float32 [slots, H, P, N]")
    _, H, P, N = state.shape
    if not (N <= 256):
        raise KernelError(f"ssm_scan: d_state {N} above 256 is not supported")
    ld_x = _rows_view(xbc, "ssm_scan: xbc")
    if not (xbc.shape[1] == H * P + 2 * n_groups * N):
        raise KernelError("ssm_scan: xbc must hold [x | B | C]")
    ld_dt = _rows_view(dt_raw, "ssm_scan: dt")
    if not (dt_raw.shape[1] == H and dt_raw.dtype == xbc.dtype):
        raise KernelError("ssm_scan: dt must be [T, H]")
    for v, nm in ((dt_shift, "dt_shift"), (a_log, "A_log"), (d_skip, "D")):
        _f32vec(v, H, f"ssm_scan: {nm}")
    if not (out.shape == (xbc.shape[0], H * P) and out.is_contiguous() and out.dtype == xbc.dtype):
        raise KernelError("ssm_scan: out must be [T, H*P]")
    zp, ld_z, zs, zb = _gate_args(gate, out, "ssm_scan")
    _call("pmm_ssm_scan_seq", xbc.data_ptr(), ld_x, dt_raw.data_ptr(), ld_dt, float(dt_scale),
          dt_shift.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), cu.data_ptr(),
          slots.data_ptr(), out.data_ptr(), n_seq, H, P, N, n_groups, zp, ld_z, zs, zb, 2 if only_single else int(bool(one_token)),
          _dt(xbc), _stream())


SSD_CHUNK = 64  # tokens per chunk of the tensor-core scan


def ssd_supported(d_head: int, d_state: int) -> bool:
    """Whether the chunked tensor-core scan is compiled for this head size / state size."""
    return bool(_fn("pmm_ssd_supported")(d_head, d_state))


def ssd_chunks(new_lens: Sequence[int]) -> int:
    return sum((n + SSD_CHUNK - 1) // SSD_CHUNK for n in new_lens)


def ssd_scratch_floats(new_lens: Sequence[int], n_heads: int, d_head: int, d_state: int,
                       n_groups: Optional[int] = None) -> int:
    """Floats of scratch for the chunked scan: every chunk's local state (float), its decay, its
    start state (bfloat16, on a 16-byte boundary) and the 64 x 64 products C.B of every
    (chunk, group); without ``n_groups`` enough for one group per head."""
    chunks = ssd_chunks(new_lens)
    per_state = chunks * n_heads * d_head * d_state
    decays = (chunks * n_heads + 3) // 4 * 4
    starts = ((per_state + 1) // 2 + 3) // 4 * 4
    return per_state + decays + starts + chunks * (n_groups or n_heads) * 64 * 64


def ssm_scan_chunked(xbc: Tensor, dt_raw: Tensor, dt_scale: float, dt_shift: Tensor, a_log: Tensor,
                     d_skip: Tensor, state: Tensor, cu: Tensor, slots: Tensor, new_lens: Sequence[int],
                     out: Tensor, n_groups: int, scratch: Tensor, gate=None) -> None:
    """The Mamba2 recurrence over prompt portions in chunks of 64 tokens on tensor cores
    (bfloat16 activations); same contract as ssm_scan_seq.  ``scratch``: float32, at least
    ssd_scratch_floats(...) elements."""
    _cuda(xbc, dt_raw, dt_shift, a_log, d_skip, state, cu, slots, out, scratch)
    if not (state.dtype == torch.float32 and state.dim() == 4 and state.is_contiguous()):
        raise KernelError("ssm_scan: state must be contiguous float32 [slots, H, P, N]")
    _, H, P, N = state.shape
    if not (xbc.dtype == torch.bfloat16 and ssd_supported(P, N)):
        raise KernelError(f"ssm_scan_chunked: needs bfloat16 and a compiled (d_head, d_state) pair, got {xbc.dtype} "
                          f"({P}, {N})")
    ld_x = _rows_view(xbc, "ssm_scan: xbc")
    if not (xbc.shape[1] == H * P + 2 * n_groups * N and ld_x % 8 == 0 and xbc.data_ptr() % 16 == 0):
        raise KernelError("ssm_scan_chunked: xbc must hold [x | B | C] in rows that start on 16-byte boundaries")
    ld_dt = _rows_view(dt_raw, "ssm_scan: dt")
    if not (dt_raw.shape[1] == H and dt_raw.dtype == xbc.dtype):
        raise KernelError("ssm_scan: dt must be [T, H]")
    for v, nm in ((dt_shift, "dt_shift"), (a_log, "A_log"), (d_skip, "D")):
        _f32vec(v, H, f"ssm_scan: {nm}")
    if not (out.shape == (xbc.shape[0], H * P) and out.is_contiguous() and out.dtype == xbc.dtype):
        raise KernelError("ssm_scan: out must be [T, H*P]")
    n_chunks = ssd_chunks(new_lens)
    need = ssd_scratch_floats(new_lens, H, P, N, n_groups)
    if not (scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need
            and scratch.data_ptr() % 16 == 0):
        raise KernelError(f"ssm_scan_chunked: needs {need} floats of 16-byte aligned scratch")
    chunk_state = scratch.data_ptr()
    chunk_decay = chunk_state + 4 * n_chunks * H * P * N
    start_state = chunk_decay + 4 * ((n_chunks * H + 3) // 4 * 4)
    chunk_cb = start_state + 4 * (((n_chunks * H * P * N + 1) // 2 + 3) // 4 * 4)
    zp, ld_z, zs, zb = _gate_args(gate, out, "ssm_scan_chunked")
    if not (zp is None or (ld_z % 2 == 0 and zp % 4 == 0)):
        raise KernelError("ssm_scan_chunked: z rows must be 4-byte aligned")
    _call("pmm_ssd_chunked", xbc.data_ptr(), ld_x, dt_raw.data_ptr(), ld_dt, float(dt_scale),
          dt_shift.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), cu.data_ptr(),
          slots.data_ptr(), out.data_ptr(), chunk_state, chunk_decay, start_state, chunk_cb, len(new_lens), n_chunks,
          H, P, N,
          n_groups, zp, ld_z, zs, zb, _stream())


SSD_TC_CHUNK = 128  # tokens per chunk of the tcgen05 scan


def ssd_tc_supported(d_head: int, d_state: int) -> bool:
    """Whether the tcgen05 scan takes this head size / state size (multiples of 16 up to 128 / 256)."""
    return bool(_fn("pmm_ssd_tc_supported")(d_head, d_state))


def ssd_tc_scratch_floats(new_lens: Sequence[int], n_heads: int, d_head: int, d_state: int) -> int:
    """Floats of scratch for the tcgen05 scan: every 128-token chunk's local state (float), its
    decay, delta and cs of its tokens per head, and its start state (bfloat16, on a 16-byte boundary)."""
    chunks = sum((n + SSD_TC_CHUNK - 1) // SSD_TC_CHUNK for n in new_lens)
    per_state = chunks * n_heads * d_head * d_state
    return (per_state + (chunks * n_heads + 3) // 4 * 4 + chunks * n_heads * 2 * SSD_TC_CHUNK
            + ((per_state + 1) // 2 + 3) // 4 * 4)


def ssm_scan_tc(xbc: Tensor, dt_raw: Tensor, dt_scale: float, dt_shift: Tensor, a_log: Tensor, d_skip: Tensor,
                state: Tensor, cu: Tensor, slots: Tensor, new_lens: Sequence[int], out: Tensor, n_groups: int,
                scratch: Tensor, gate=None, skip_single: bool = False) -> None:
    """The Mamba2 recurrence over prompt portions in chunks of 128 tokens on the tcgen05 tensor
    cores (bfloat16 activations); same contract as ssm_scan_seq.  ``scratch``: float32, at least
    ssd_tc_scratch_floats(...) elements.  ``skip_single``: sequences that bring exactly one token are
    left alone (their rows of ``out`` and their states): ssm_scan_seq(only_single=True) takes them."""
    _cuda(xbc, dt_raw, dt_shift, a_log, d_skip, state, cu, slots, out, scratch)
    if not (state.dtype == torch.float32 and state.dim() == 4 and state.is_contiguous()):
        raise KernelError("ssm_scan: state must be contiguous float32 [slots, H, P, N]")
    _, H, P, N = state.shape
    if not (xbc.dtype == torch.bfloat16 and ssd_tc_supported(P, N)):
        raise KernelError(f"ssm_scan_tc: needs bfloat16, a head size that is a multiple of 16 up to 128 and a state size that is a "
                          f"multiple of 16 up to 256, got {xbc.dtype} ({P}, {N})")
    ld_x = _rows_view(xbc, "ssm_scan: xbc")
    if not (xbc.shape[1] == H * P + 2 * n_groups * N and ld_x % 8 == 0 and xbc.data_ptr() % 16 == 0):
        raise KernelError("ssm_scan_tc: xbc must hold [x | B | C] in rows that start on 16-byte boundaries")
    ld_dt = _rows_view(dt_raw, "ssm_scan: dt")
    if not (dt_raw.shape[1] == H and dt_raw.dtype == xbc.dtype):
        raise KernelError("ssm_scan: dt must be [T, H]")
    for v, nm in ((dt_shift, "dt_shift"), (a_log, "A_log"), (d_skip, "D")):
        _f32vec(v, H, f"ssm_scan: {nm}")
    if not (out.shape == (xbc.shape[0], H * P) and out.is_contiguous() and out.dtype == xbc.dtype
            and out.data_ptr() % 16 == 0):
        raise KernelError("ssm_scan: out must be [T, H*P] on a 16-byte boundary")
    n_chunks = sum((n + SSD_TC_CHUNK - 1) // SSD_TC_CHUNK for n in new_lens)
    need = ssd_tc_scratch_floats(new_lens, H, P, N)
    if not (scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need
            and scratch.data_ptr() % 16 == 0):
        raise KernelError(f"ssm_scan_tc: needs {need} floats of 16-byte aligned scratch")
    chunk_state = scratch.data_ptr()
    chunk_decay = chunk_state + 4 * n_chunks * H * P * N
    chunk_dt = chunk_decay + 4 * ((n_chunks * H + 3) // 4 * 4)
    start_state = chunk_dt + 4 * n_chunks * H * 2 * SSD_TC_CHUNK
    zp, ld_z, zs, zb = _gate_args(gate, out, "ssm_scan_tc")
    n_multi = getattr(new_lens, "multi", None)  # lengths given as bounds carry the bound with them
    if n_multi is None:
        n_multi = sum(1 for n in new_lens if n > 1)
    _call("pmm_ssd_tc", xbc.data_ptr(), ld_x, dt_raw.data_ptr(), ld_dt, float(dt_scale), dt_shift.data_ptr(),
          a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), cu.data_ptr(), slots.data_ptr(), out.data_ptr(),
          chunk_state, chunk_decay, chunk_dt, start_state, len(new_lens), n_chunks, H, P, N, n_groups, zp, ld_z, zs, zb,
          int(bool(skip_single)), n_multi if skip_single else 0,
          _tc_status(xbc.device).data_ptr(), _stream())


def gated_norm(y: Tensor, z_raw: Tensor, z_scale: float, z_bias: Optional[Tensor],
               weight: Optional[Tensor], eps: float, n_groups: int, norm_before_gate: bool,
               out: Tensor, gate: str = "silu") -> None:
    """out = y*silu(z), optionally RMS-normalised per group of channels (before or after the gate).
    ``gate`` "sigmoid": sigmoid(z) in place of silu(z).  y may be float32 whatever the type of z and
    out (a recurrence's output); out may be a column block of a wider matrix."""
    _cuda(y, z_raw, z_bias, weight, out)
    T, I = y.shape
    if not (y.is_contiguous() and out.dim() == 2 and out.stride(1) == 1 and out.shape == y.shape
            and y.dtype in (out.dtype, torch.float32)):
        raise KernelError("gated_norm: y contiguous [T, I], out [T, I] with unit column stride; y of out's type or float32")
    if gate not in ("silu", "sigmoid"):
        raise KernelError("gated_norm: the gate is 'silu' or 'sigmoid'")
    ld_z = _rows_view(z_raw, "gated_norm: z")
    if not (z_raw.shape == y.shape and z_raw.dtype == out.dtype):
        raise KernelError("gated_norm: z must match out")
    _f32vec(z_bias, I, "gated_norm: z_bias")
    _f32vec(weight, I, "gated_norm: weight")
    groups = n_groups if weight is not None else 1
    if not (I % groups == 0):
        raise KernelError("gated_norm: width must be a multiple of the group count")
    _call("pmm_gated_norm", y.data_ptr(), z_raw.data_ptr(), ld_z, float(z_scale), _ptr(z_bias),
          _ptr(weight), float(eps), int(bool(norm_before_gate)), out.data_ptr(), out.stride(0), T, I, groups, _dt(out),
          int(y.dtype == torch.float32 and out.dtype != torch.float32), int(gate == "sigmoid"), _stream())


def check_head_dim(head_dim: int, limit: int = 256) -> None:
    """Head sizes the attention kernels take: up to 256 on the tensor cores; the float kernel, which every
    other size falls to, up to ``FLOAT_ATTENTION_MAX_HEAD`` (the rows of wide latents)."""
    if not (head_dim % 16 == 0 and 16 <= head_dim <= limit):
        raise KernelError(f"attention kernels take head sizes 16..{limit} in steps of 16, got {head_dim}")


FLOAT_ATTENTION_MAX_HEAD = 512


def qkv_rope_store(q: Tensor, k: Optional[Tensor], v: Optional[Tensor], q_scale: float, k_scale: float,
                   v_scale: float, inv_freq: Optional[Tensor], positions: Tensor, seq_of: Tensor,
                   block_table: Optional[Tensor], pool: Optional[Tensor], q_out: Tensor,
                   k_out: Optional[Tensor], v_out: Optional[Tensor], n_q_heads: int, n_kv_heads: int,
                   head_dim: int) -> None:
    """Scales q/k/v, rotates q and k (when inv_freq is given) and stores k/v into the pages of
    ``pool`` [pages, 2, page_size, Hkv*Dh] through ``block_table`` [n_seq, max_blocks], or into
    k_out/v_out when no pool is given.  With k and v None (n_kv_heads 0) only q is prepared."""
    _cuda(q, k, v, inv_freq, positions, seq_of, block_table, pool, q_out, k_out, v_out)
    check_head_dim(head_dim)
    T = q.shape[0]
    ldq = _rows_view(q, "qkv: q")
    if not (q.shape[1] == n_q_heads * head_dim and q.dtype == q_out.dtype):
        raise KernelError("qkv: q width or type")
    if not (q_out.is_contiguous() and q_out.shape == (T, n_q_heads * head_dim)):
        raise KernelError("qkv: q_out must be [T, Hq*Dh]")
    _f32vec(inv_freq, head_dim // 2, "qkv: inv_freq")
    _i32(positions, "qkv: positions")
    _i32(seq_of, "qkv: seq_of")
    page_size, max_blocks, ldk, ldv = 0, 0, 0, 0
    if k is None or v is None:
        if not (k is None and v is None and n_kv_heads == 0):
            raise KernelError("qkv: queries only means no k, no v, no kv heads")
        pool = block_table = k_out = v_out = None
    else:
        ldk, ldv = _rows_view(k, "qkv: k"), _rows_view(v, "qkv: v")
        kv_dim = n_kv_heads * head_dim
        if not (k.shape[1] == kv_dim and v.shape[1] == kv_dim and q.dtype == k.dtype == v.dtype):
            raise KernelError("qkv: slice widths do not match the head counts")
        if pool is not None:
            if not (block_table is not None):
                raise KernelError("qkv: a pool needs a block table")
            _i32(block_table, "qkv: block_table")
            if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == kv_dim and pool.is_contiguous()
                    and pool.dtype == q.dtype):
                raise KernelError("qkv: pool must be contiguous [pages, 2, page_size, Hkv*Dh]")
            page_size, max_blocks = pool.shape[2], block_table.shape[1]
        else:
            if not (k_out is not None and v_out is not None and k_out.is_contiguous() and v_out.is_contiguous()
                    and k_out.shape == (T, kv_dim) and v_out.shape == (T, kv_dim)):
                raise KernelError("qkv: k_out/v_out must be [T, Hkv*Dh]")
    _call("pmm_qkv_rope_store", q.data_ptr(), ldq, _ptr(k), ldk, _ptr(v), ldv, float(q_scale),
          float(k_scale), float(v_scale), _ptr(inv_freq), positions.data_ptr(), seq_of.data_ptr(),
          _ptr(block_table), max_blocks, _ptr(pool), page_size, q_out.data_ptr(), _ptr(k_out),
          _ptr(v_out), T, n_q_heads, n_kv_heads, head_dim, _dt(q), _stream())


def kv_store(k: Tensor, v: Tensor, positions: Tensor, seq_of: Tensor, block_table: Tensor,
             pool: Tensor) -> None:
    """Copies contiguous k/v rows [T, Hkv*Dh] into the pages of ``pool``."""
    _cuda(k, v, positions, seq_of, block_table, pool)
    T, kv_dim = k.shape
    if not (k.is_contiguous() and v.is_contiguous() and v.shape == k.shape and k.dtype == v.dtype == pool.dtype):
        raise KernelError("kv_store: k and v must be contiguous [T, Hkv*Dh] of the pool's type")
    if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == kv_dim and pool.is_contiguous()):
        raise KernelError("kv_store: pool must be contiguous [pages, 2, page_size, Hkv*Dh]")
    _i32(block_table, "kv_store: block_table")
    _call("pmm_kv_store", k.data_ptr(), v.data_ptr(), positions.data_ptr(), seq_of.data_ptr(),
          block_table.data_ptr(), block_table.shape[1], pool.data_ptr(), pool.shape[2], T, kv_dim,
          _dt(k), _stream())


def attention_scratch_floats(T: int, n_q_heads: int, head_dim: int, n_splits: int) -> int:
    return T * n_q_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0


def flash_supported(n_q_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core attention kernel takes this shape (bfloat16 caches only)."""
    return bool(_fn("pmm_flash_supported")(n_q_heads, n_kv_heads, head_dim))


def flash_tile_rows(n_q_heads: int, n_kv_heads: int, head_dim: int, new_lens: Sequence[int]) -> int:
    """Rows of (token, query head of a group) that one block of the tensor-core attention kernel
    takes: 16 when every sequence brings at most 16 of them (decode), 128 for long portions of
    head sizes up to 64 (each key/value fragment then feeds two row tiles), else 64."""
    group = n_q_heads // n_kv_heads
    if group <= 16 and max(new_lens) * group <= 16:
        return 16
    if head_dim <= 64 and sum(new_lens) * n_q_heads >= _FLASH_128_FROM_ROWS:
        return 128
    return 64


_FLASH_128_FROM_ROWS = 49152  # measured: 64 rows a block are faster at 16k rows, 128 at 64k


def paged_attention(q: Tensor, pool: Tensor, block_table: Tensor, positions: Tensor, seq_of: Tensor,
                    out: Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, softmax_scale: float,
                    window: int = 0, n_splits: int = 1, split_len: int = 0,
                    scratch: Optional[Tensor] = None, cu_seqlens: Optional[Tensor] = None,
                    new_lens: Optional[Sequence[int]] = None, use_tensor_cores: bool = True,
                    split_counter: Optional[Tensor] = None, tile_rows: Optional[int] = None,
                    sink: Optional[Tensor] = None, keep_first: int = 0, lse: Optional[Tensor] = None) -> None:
    """Causal attention of every token over keys lo..pos of its request in the paged cache.
    ``keep_first``: the request's first keep_first keys stay visible behind a window (at their true positions).
    The float kernel walks both key ranges itself; the tensor-core kernel takes them with one key split and
    ``lse`` (float32 [T, Hq, 2] scratch): it leaves every row's maximum and sum there and `kept_first_merge` adds
    the kept keys.
    ``sink`` (one float per query head): the softmax's denominator also holds exp(sink[h]), a score
    without key or value.
    With ``cu_seqlens`` and ``new_lens`` (tokens per sequence, host values) a bfloat16 cache of a
    supported shape goes to the tensor-core kernel; everything else to the float kernel.
    ``split_counter`` (int32, zero between calls, at least tiles x kv heads entries) lets the
    tensor-core kernel merge its key splits itself instead of in a second launch.  ``tile_rows``
    (rows of (token, query head of a group) per block: 16, 64 or 128) defaults to flash_tile_rows."""
    _cuda(q, pool, block_table, positions, seq_of, out, scratch, cu_seqlens)
    check_head_dim(head_dim, FLOAT_ATTENTION_MAX_HEAD)
    T = q.shape[0]
    if not (q.is_contiguous() and out.is_contiguous() and q.shape == (T, n_q_heads * head_dim)
            and out.shape == q.shape and q.dtype == out.dtype == pool.dtype):
        raise KernelError("attention: q and out must be contiguous [T, Hq*Dh] of the pool's type")
    if not (n_q_heads % n_kv_heads == 0):
        raise KernelError("attention: query heads must be a multiple of key/value heads")
    if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == n_kv_heads * head_dim
            and pool.is_contiguous()):
        raise KernelError("attention: pool must be contiguous [pages, 2, page_size, Hkv*Dh]")
    _i32(block_table, "attention: block_table")
    _i32(positions, "attention: positions")
    _i32(seq_of, "attention: seq_of")
    part_o = part_ml = None
    if n_splits > 1:
        need = attention_scratch_floats(T, n_q_heads, head_dim, n_splits)
        if not (scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
                and scratch.numel() >= need):
            raise KernelError(f"attention: split keys need {need} floats of scratch")
        if not (split_len > 0 and split_len % 32 == 0):
            raise KernelError("attention: split_len must be a positive multiple of 32")
        part_o = scratch.data_ptr()
        part_ml = part_o + 4 * T * n_q_heads * n_splits * head_dim
    _f32vec(sink, n_q_heads, "attention: sink")
    if not (keep_first >= 0):
        raise KernelError("attention: keep_first must not be negative")
    flash = (use_tensor_cores and q.dtype == torch.bfloat16 and cu_seqlens is not None and new_lens is not None
             and flash_supported(n_q_heads, n_kv_heads, head_dim)
             and (keep_first == 0 or window == 0 or (lse is not None and n_splits == 1)))
    keep = int(keep_first) if window > 0 else 0
    if flash:
        _i32(cu_seqlens, "attention: cu_seqlens")
        group = n_q_heads // n_kv_heads
        if tile_rows is None:
            tile_rows = flash_tile_rows(n_q_heads, n_kv_heads, head_dim, new_lens)
        if not (tile_rows in (16, 64, 128) and group <= tile_rows and (tile_rows < 128 or head_dim <= 64)
                and (tile_rows > 16 or max(new_lens) * group <= 16)):
            raise KernelError(f"attention: {tile_rows} rows per block do not fit this shape")
        tokens_per_tile = tile_rows // group
        n_tiles = sum((n + tokens_per_tile - 1) // tokens_per_tile for n in new_lens)
        counter = None
        if (split_counter is not None and 1 < n_splits <= 64 and split_counter.numel() >= n_tiles * n_kv_heads):
            _cuda(split_counter)
            _i32(split_counter, "attention: split_counter")
            counter = split_counter.data_ptr()
        _call("pmm_flash_paged_attention", q.data_ptr(), pool.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], positions.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(), part_o,
              part_ml, float(softmax_scale), int(window), int(split_len), int(n_splits), pool.shape[2],
              len(new_lens), n_tiles, int(tile_rows), n_q_heads, n_kv_heads, head_dim, counter, _ptr(sink),
              _lse_ptr(lse, T, n_q_heads) if keep > 0 else None, _stream())
        if keep > 0:
            kept_first_merge(q, pool, block_table, positions, seq_of, out, lse, n_q_heads, n_kv_heads, head_dim,
                             softmax_scale, window, keep)
        if counter is not None:
            return
    else:
        _call("pmm_paged_attention", q.data_ptr(), pool.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], positions.data_ptr(), seq_of.data_ptr(), out.data_ptr(), part_o, part_ml,
              float(softmax_scale), int(window), int(split_len), int(n_splits), pool.shape[2], T, n_q_heads,
              n_kv_heads, head_dim, _dt(q), _ptr(sink), keep, _stream())
    if n_splits > 1:
        _call("pmm_flash_combine", part_o, part_ml, out.data_ptr(), T * n_q_heads, int(n_splits), head_dim,
              _dt(out), _stream())


def _lse_ptr(lse: Optional[Tensor], T: int, n_q_heads: int) -> int:
    if not (lse is not None and lse.is_cuda and lse.dtype == torch.float32 and lse.is_contiguous()
            and lse.numel() >= 2 * T * n_q_heads):
        raise KernelError("attention: kept first keys need float32 scratch [T, Hq, 2] for the rows' maxima and sums")
    return lse.data_ptr()


def kept_first_merge(q: Tensor, pool: Tensor, block_table: Tensor, positions: Tensor, seq_of: Tensor, out: Tensor,
                     lse: Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, softmax_scale: float, window: int,
                     keep_first: int) -> None:
    """``out`` [T, Hq*Dh] holds every row's attention over its window (and sink), ``lse`` [T, Hq, 2] that result's
    maximum score and sum of exponentials: the request's first ``keep_first`` keys that a row's window has left
    behind are added, and the row becomes the softmax over both sets of keys."""
    _cuda(q, pool, block_table, positions, seq_of, out, lse)
    T = q.shape[0]
    if not (q.is_contiguous() and out.is_contiguous() and q.shape == (T, n_q_heads * head_dim) and out.shape == q.shape
            and q.dtype == out.dtype == pool.dtype):
        raise KernelError("kept_first_merge: q and out must be contiguous [T, Hq*Dh] of the pool's type")
    if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == n_kv_heads * head_dim and pool.is_contiguous()):
        raise KernelError("kept_first_merge: pool must be contiguous [pages, 2, page_size, Hkv*Dh]")
    _i32(block_table, "kept_first_merge: block_table")
    _i32(positions, "kept_first_merge: positions")
    _i32(seq_of, "kept_first_merge: seq_of")
    _call("pmm_kept_first_merge", q.data_ptr(), pool.data_ptr(), block_table.data_ptr(), block_table.shape[1],
          positions.data_ptr(), seq_of.data_ptr(), out.data_ptr(), _lse_ptr(lse, T, n_q_heads), float(softmax_scale),
          int(window), int(keep_first), pool.shape[2], T, n_q_heads, n_kv_heads, head_dim, _dt(q), _stream())


# Decode attention with TMA tile loads where the sizes allow (PMM_TMA_DECODE=0: cp.async gathers throughout).
_TMA_DECODE = os.environ.get("PMM_TMA_DECODE", "1") == "1"


def flash_decode_supported(n_q_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether flash_decode_attention takes this head shape (bfloat16, at most 16 query heads a group)."""
    return flash_supported(n_q_heads, n_kv_heads, head_dim) and n_q_heads // n_kv_heads <= 16


def flash_decode_attention(q: Tensor, k: Optional[Tensor], v: Optional[Tensor], q_scale: float, k_scale: float,
                           v_scale: float, inv_freq: Optional[Tensor], pool: Tensor, block_table: Tensor,
                           positions: Tensor, out: Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int,
                           softmax_scale: float, window: int = 0, n_splits: int = 1, split_len: int = 0,
                           scratch: Optional[Tensor] = None, split_counter: Optional[Tensor] = None,
                           sink: Optional[Tensor] = None, keep_first: int = 0, lse: Optional[Tensor] = None,
                           seq_of: Optional[Tensor] = None) -> None:
    """A decode step's attention straight from the projections (token t is sequence t's one new
    token): scales and rotates queries and new keys, writes the new keys and values into their
    cache pages and attends over the cache, in one launch.  ``k``/``v`` None: the cache has them.
    ``sink``: see paged_attention.  ``keep_first`` > 0 behind a window: one key split, ``lse`` scratch and
    ``seq_of`` (token -> sequence, here 0, 1, 2, ...), and queries that are rotated already (k and v None)."""
    _cuda(q, k, v, inv_freq, pool, block_table, positions, out, scratch, split_counter, sink)
    keep = int(keep_first) if window > 0 else 0
    lse_ptr = None
    if keep > 0:
        if not (n_splits == 1 and k is None and v is None and inv_freq is None and seq_of is not None
                and q_scale == 1.0 and q.is_contiguous()):
            raise KernelError("decode attention: kept first keys take one key split and prepared queries")
        lse_ptr = _lse_ptr(lse, q.shape[0], n_q_heads)
    _f32vec(sink, n_q_heads, "decode attention: sink")
    n_seq = q.shape[0]
    kv_dim = n_kv_heads * head_dim
    if not (q.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and flash_decode_supported(n_q_heads, n_kv_heads, head_dim)):
        raise KernelError("decode attention: bfloat16 and a supported shape")
    ldq = _rows_view(q, "decode attention: q")
    if not (q.shape[1] == n_q_heads * head_dim and out.is_contiguous() and out.shape == (n_seq, n_q_heads * head_dim)):
        raise KernelError("decode attention: q/out must be [n_seq, Hq*Dh]")
    ldk = ldv = 0
    if k is not None or v is not None:
        if not (k is not None and v is not None and k.dtype == v.dtype == torch.bfloat16
                and k.shape == (n_seq, kv_dim) and v.shape == (n_seq, kv_dim)):
            raise KernelError("decode attention: k/v must be [n_seq, Hkv*Dh]")
        ldk, ldv = _rows_view(k, "decode attention: k"), _rows_view(v, "decode attention: v")
    _f32vec(inv_freq, head_dim // 2, "decode attention: inv_freq")
    if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == kv_dim and pool.is_contiguous()):
        raise KernelError("decode attention: pool must be contiguous [pages, 2, page_size, Hkv*Dh]")
    _i32(block_table, "decode attention: block_table")
    _i32(positions, "decode attention: positions")
    if not (block_table.shape[0] >= n_seq and positions.numel() >= n_seq):
        raise KernelError("decode attention: one table row and position per sequence")
    part_o = part_ml = counter = None
    if n_splits > 1:
        need = attention_scratch_floats(n_seq, n_q_heads, head_dim, n_splits)
        if not (scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
                and scratch.numel() >= need):
            raise KernelError(f"decode attention: split keys need {need} floats of scratch")
        if not (split_len > 0 and split_len % 32 == 0 and n_splits <= 64):
            raise KernelError("decode attention: bad key split")
        if not (split_counter is not None and split_counter.numel() >= n_seq * n_kv_heads):
            raise KernelError("decode attention: split keys need a counter per (sequence, key/value head)")
        _i32(split_counter, "decode attention: split_counter")
        part_o = scratch.data_ptr()
        part_ml = part_o + 4 * n_seq * n_q_heads * n_splits * head_dim
        counter = split_counter.data_ptr()
    if (_TMA_DECODE and (n_splits == 1 or split_len % 64 == 0)
            and _fn("pmm_decode_attention_tma_supported")(n_q_heads, n_kv_heads, head_dim, pool.shape[2])):
        # the copy engine brings the tiles (pages of a multiple of 64 positions, head sizes 64 and 128)
        _call("pmm_decode_attention_tma", q.data_ptr(), ldq, _ptr(k), ldk, _ptr(v), ldv, float(q_scale), float(k_scale),
              float(v_scale), _ptr(inv_freq), pool.data_ptr(), pool.shape[0], block_table.data_ptr(),
              block_table.shape[1], positions.data_ptr(), out.data_ptr(), part_o, part_ml, float(softmax_scale),
              int(window), int(split_len), int(n_splits), pool.shape[2], n_seq, n_q_heads, n_kv_heads, head_dim, counter,
              _tc_status(q.device).data_ptr(), _ptr(sink), lse_ptr, _stream())
        if keep > 0:
            kept_first_merge(q, pool, block_table, positions, seq_of, out, lse, n_q_heads, n_kv_heads, head_dim,
                             softmax_scale, window, keep)
        return
    _call("pmm_flash_decode_attention", q.data_ptr(), ldq, _ptr(k), ldk, _ptr(v), ldv, float(q_scale), float(k_scale),
          float(v_scale), _ptr(inv_freq), pool.data_ptr(), block_table.data_ptr(), block_table.shape[1],
          positions.data_ptr(), out.data_ptr(), part_o, part_ml, float(softmax_scale), int(window), int(split_len),
          int(n_splits), pool.shape[2], n_seq, n_q_heads, n_kv_heads, head_dim, counter, _ptr(sink), lse_ptr, _stream())
    if keep > 0:
        kept_first_merge(q, pool, block_table, positions, seq_of, out, lse, n_q_heads, n_kv_heads, head_dim,
                         softmax_scale, window, keep)


SKINNY_MAX_TOKENS = 64  # the weight-streaming products take up to 64 tokens (where their shared memory fits)
SKINNY_NORM_MAX_TOKENS = 16  # every block redoes the norm of all rows: beyond this a norm launch of its own is cheaper
# from here on the tcgen05 form (skinny_tc_*) is the faster one inside a decode step (0.5B sizes, ms a step,
# mma.sync / tcgen05: 32 tokens 1.87 / 2.09, 40 tokens 2.35 / 2.26, 48 tokens 2.63 / 2.51); PMM_TC_SKINNY_FROM moves it
SKINNY_TC_FROM_TOKENS = int(os.environ.get("PMM_TC_SKINNY_FROM", "33"))
SKINNY_NORM_MAX_WIDTH = 1024  # ... and so it is for rows wider than a warp keeps in registers (they are read twice)


def _skinny_check(M: int, w: Tensor, K: int, what: str) -> None:
    if not (M <= 64):
        raise KernelError(f"{what}: at most 64 tokens")
    if not (w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous() and w.shape[1] == K and K % 8 == 0):
        raise KernelError(f"{what}: weights must be contiguous bfloat16 [rows, K] with K a multiple of 8")


def skinny_fits(M: int, K: int) -> bool:
    """Whether M tokens x K columns of activations fit in shared memory beside the weight pipeline
    (the products that cannot split K keep the whole row block resident)."""
    mp = 8 if M <= 8 else 16 if M <= 16 else 32 if M <= 32 else 64
    kx = (K + 255) // 256 * 256
    stages = 3 if mp > 32 else 5
    return M <= 64 and stages * 32 * 264 * 2 + mp * (kx + 8) * 2 + 3 * 32 * mp * 4 + (kx + mp) * 4 <= 220 * 1024


def skinny_linear_norm(h: Tensor, norm_weight: Tensor, eps: float, weight: Tensor, out: Tensor) -> None:
    """out[M, N] = (rmsnorm(h) * norm_weight) @ weight^T for M <= 64 rows of the float32 stream."""
    _cuda(h, norm_weight, weight, out)
    M, K = h.shape
    if not (h.dtype == torch.float32 and h.is_contiguous()):
        raise KernelError("skinny_linear_norm: h must be contiguous float32")
    _skinny_check(M, weight, K, "skinny_linear_norm")
    if not (skinny_fits(M, K)):
        raise KernelError(f"skinny_linear_norm: {M} tokens x {K} columns do not fit in shared memory")
    _f32vec(norm_weight, K, "skinny_linear_norm: norm weight")
    N = weight.shape[0]
    if not (out.dtype == torch.bfloat16 and out.shape == (M, N) and out.stride(1) == 1):
        raise KernelError("skinny_linear_norm: out [M, N] bfloat16")
    _call("pmm_skinny_gemm", 0, M, N, None, 0, h.data_ptr(), norm_weight.data_ptr(), float(eps), weight.data_ptr(), K,
          1.0, None, 0, None, 0, 0.0, out.data_ptr(), out.stride(0), None, 1, _stream())


def _skinny_x(x: Tensor, M: int, K: int, what: str) -> None:
    if not (x.dtype == torch.bfloat16 and x.shape == (M, K) and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0):
        raise KernelError(f"{what}: x must be bfloat16 [M, K] with 16-byte aligned rows")


def skinny_linear(x: Tensor, weight: Tensor, out: Tensor) -> None:
    """out[M, N] = x @ weight^T for M <= 64 rows of bfloat16 activations (weights streamed once)."""
    _cuda(x, weight, out)
    M, K = x.shape
    _skinny_check(M, weight, K, "skinny_linear")
    _skinny_x(x, M, K, "skinny_linear")
    if not (skinny_fits(M, K)):
        raise KernelError(f"skinny_linear: {M} tokens x {K} columns do not fit in shared memory")
    N = weight.shape[0]
    if not (out.dtype == torch.bfloat16 and out.shape == (M, N) and out.stride(1) == 1):
        raise KernelError("skinny_linear: out [M, N] bfloat16")
    _call("pmm_skinny_gemm", 0, M, N, x.data_ptr(), x.stride(0), None, None, 0.0, weight.data_ptr(), K,
          1.0, None, 0, None, 0, 0.0, out.data_ptr(), out.stride(0), None, 1, _stream())


def skinny_linear_f32(x: Tensor, weight: Tensor, out: Tensor, scale: float) -> None:
    """out[M, N] (float32) = scale * (x @ weight^T) for M <= 64 rows of bfloat16 activations: the
    output head of a step that asks for few rows of logits (the table is streamed once)."""
    _cuda(x, weight, out)
    M, K = x.shape
    _skinny_check(M, weight, K, "skinny_linear_f32")
    _skinny_x(x, M, K, "skinny_linear_f32")
    if not (skinny_fits(M, K)):
        raise KernelError(f"skinny_linear_f32: {M} tokens x {K} columns do not fit in shared memory")
    N = weight.shape[0]
    if not (out.dtype == torch.float32 and out.shape == (M, N) and out.stride(1) == 1):
        raise KernelError("skinny_linear_f32: out [M, N] float32")
    _call("pmm_skinny_gemm_f32out", M, N, x.data_ptr(), x.stride(0), weight.data_ptr(), K, float(scale),
          out.data_ptr(), out.stride(0), _stream())


def skinny_swiglu(x: Tensor, gate_up: Tensor, gate_mult: float, out: Tensor) -> None:
    """out[M, F] = silu(gate * gate_mult) * up with [gate | up] = x @ gate_up^T, x bfloat16."""
    _cuda(x, gate_up, out)
    M, K = x.shape
    _skinny_check(M, gate_up, K, "skinny_swiglu")
    _skinny_x(x, M, K, "skinny_swiglu")
    if not (skinny_fits(M, K)):
        raise KernelError(f"skinny_swiglu: {M} tokens x {K} columns do not fit in shared memory")
    F = gate_up.shape[0] // 2
    if not (gate_up.shape[0] == 2 * F and out.dtype == torch.bfloat16 and out.shape == (M, F) and out.is_contiguous()):
        raise KernelError("skinny_swiglu: out [M, F] bfloat16 for gate_up [2F, K]")
    _call("pmm_skinny_gemm", 1, M, F, x.data_ptr(), x.stride(0), None, None, 0.0, gate_up.data_ptr(), K,
          float(gate_mult), None, 0, None, 0, 0.0, out.data_ptr(), out.stride(0), None, 1, _stream())


def skinny_swiglu_norm(h: Tensor, norm_weight: Tensor, eps: float, gate_up: Tensor, gate_mult: float,
                       out: Tensor) -> None:
    """out[M, F] = silu(gate * gate_mult) * up with [gate | up] = (rmsnorm(h) * norm_weight) @ gate_up^T."""
    _cuda(h, norm_weight, gate_up, out)
    M, K = h.shape
    if not (h.dtype == torch.float32 and h.is_contiguous()):
        raise KernelError("skinny_swiglu_norm: h must be contiguous float32")
    _skinny_check(M, gate_up, K, "skinny_swiglu_norm")
    if not (skinny_fits(M, K)):
        raise KernelError(f"skinny_swiglu_norm: {M} tokens x {K} columns do not fit in shared memory")
    _f32vec(norm_weight, K, "skinny_swiglu_norm: norm weight")
    F = gate_up.shape[0] // 2
    if not (gate_up.shape[0] == 2 * F and out.dtype == torch.bfloat16 and out.shape == (M, F) and out.is_contiguous()):
        raise KernelError("skinny_swiglu_norm: out [M, F] bfloat16 for gate_up [2F, K]")
    _call("pmm_skinny_gemm", 1, M, F, None, 0, h.data_ptr(), norm_weight.data_ptr(), float(eps), gate_up.data_ptr(), K,
          float(gate_mult), None, 0, None, 0, 0.0, out.data_ptr(), out.stride(0), None, 1, _stream())


def skinny_residual(h: Tensor, products: Sequence[Tuple[Tensor, Tensor, float]]) -> None:
    """h[M, N] += sum_i scale_i * (x_i @ w_i^T) for one or two (x, w, scale); float32 atomics, the K
    ranges are split over blocks."""
    if not (1 <= len(products) <= 2):
        raise KernelError("skinny_residual: one or two products")
    M, N = h.shape
    _cuda(h)
    if not (h.dtype == torch.float32 and h.is_contiguous()):
        raise KernelError("skinny_residual: h must be contiguous float32")
    args = []
    k_max = 0
    for x, w, sc in products:
        _cuda(x, w)
        K = x.shape[1]
        if not (x.dtype == torch.bfloat16 and x.shape[0] == M and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0):
            raise KernelError("skinny_residual: x must be bfloat16 [M, K] with 16-byte aligned rows")
        _skinny_check(M, w, K, "skinny_residual")
        if not (w.shape[0] == N):
            raise KernelError("skinny_residual: weight rows must equal the stream width")
        args.append((x.data_ptr(), x.stride(0), w.data_ptr(), K, float(sc)))
        k_max = max(k_max, K)
    chunks = (k_max + 255) // 256
    col_blocks = (N + 31) // 32 * len(products)
    k_split = max(1, min(chunks, (296 + col_blocks - 1) // col_blocks))
    while k_split < chunks and not skinny_fits(M, (chunks + k_split - 1) // k_split * 256):
        k_split += 1
    a0 = args[0]
    a1 = args[1] if len(args) > 1 else (None, 0, None, 0, 0.0)
    _call("pmm_skinny_gemm", 2, M, N, a0[0], a0[1], None, None, 0.0, a0[2], a0[3], a0[4], a1[0], a1[1], a1[2], a1[3],
          a1[4], None, 0, h.data_ptr(), k_split, _stream())


class _SkinnyPhase(ctypes.Structure):
    """One product of skinny_chain; mirrors PmmSkinnyPhase of csrc/skinny_gemm.cu."""
    _fields_ = [("mode", ctypes.c_int), ("N", ctypes.c_int), ("x0", ctypes.c_void_p), ("ldx0", ctypes.c_longlong),
                ("h_in", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("eps", ctypes.c_float),
                ("w0", ctypes.c_void_p), ("K0", ctypes.c_int), ("scale0", ctypes.c_float),
                ("x1", ctypes.c_void_p), ("ldx1", ctypes.c_longlong), ("w1", ctypes.c_void_p), ("K1", ctypes.c_int),
                ("scale1", ctypes.c_float), ("y", ctypes.c_void_p), ("ldy", ctypes.c_longlong),
                ("h_out", ctypes.c_void_p)]


_CHAIN_STATE: Dict[torch.device, Tuple[Tensor, Tensor]] = {}
SKINNY_CHAIN_MAX = 4


def _chain_state(device: torch.device) -> Tuple[Tensor, Tensor]:
    st = _CHAIN_STATE.get(device)
    if st is None:
        st = (torch.zeros(1, dtype=torch.int64, device=device), _watch(device).words[1:2])
        _CHAIN_STATE[device] = st
    return st


def skinny_chain_status(device) -> int:
    """0, or 1 when a barrier wait of a skinny_chain launch on this device ever gave up (synchronises)."""
    return int(_watch(torch.device(device)).words[1].item())


def skinny_chain(h: Tensor, phases: Sequence[Tuple]) -> None:
    """Up to 4 weight-streaming products over the float32 stream ``h`` [M <= 16, D] in ONE launch,
    each reading what the one before it wrote (barriers over the grid in between, the next
    product's weights requested before each barrier).  Phases:
      ("residual", [(x, w, scale), ...])                      h += sum scale * x @ w^T      (1 or 2 products)
      ("swiglu", norm_weight, eps, gate_up, gate_mult, out)   out = silu(g * gate_mult) * u, [g|u] = norm(h) @ gate_up^T
      ("store", norm_weight, eps, weight, out)                out = norm(h) @ weight^T
    """
    _cuda(h)
    M, D = h.shape
    if not (h.dtype == torch.float32 and h.is_contiguous() and M <= 16):
        raise KernelError("skinny_chain: h must be contiguous float32 [<=16, D]")
    if not (1 <= len(phases) <= SKINNY_CHAIN_MAX):
        raise KernelError(f"skinny_chain: 1 to {SKINNY_CHAIN_MAX} phases")
    arr = (_SkinnyPhase * len(phases))()
    for ph, slot in zip(phases, arr):
        kind = ph[0]
        if kind == "residual":
            products = ph[1]
            if not (1 <= len(products) <= 2):
                raise KernelError("skinny_chain: one or two products per residual phase")
            slot.mode, slot.N, slot.h_out = 2, D, h.data_ptr()
            for i, (x, w, sc) in enumerate(products):
                _cuda(x, w)
                K = x.shape[1]
                if not (x.dtype == torch.bfloat16 and x.shape[0] == M and x.stride(1) == 1 and x.stride(0) % 8 == 0
                        and x.data_ptr() % 16 == 0):
                    raise KernelError("skinny_chain: x must be bfloat16 [M, K] with 16-byte aligned rows")
                _skinny_check(M, w, K, "skinny_chain")
                if not (w.shape[0] == D):
                    raise KernelError("skinny_chain: weight rows must equal the stream width")
                if i == 0:
                    slot.x0, slot.ldx0, slot.w0, slot.K0, slot.scale0 = x.data_ptr(), x.stride(0), w.data_ptr(), K, float(sc)
                else:
                    slot.x1, slot.ldx1, slot.w1, slot.K1, slot.scale1 = x.data_ptr(), x.stride(0), w.data_ptr(), K, float(sc)
        elif kind in ("swiglu", "store"):
            norm_w, eps, w = ph[1], ph[2], ph[3]
            out = ph[-1]
            _cuda(norm_w, w, out)
            _skinny_check(M, w, D, "skinny_chain")
            if not (skinny_fits(M, D)):
                raise KernelError(f"skinny_chain: {M} tokens x {D} columns do not fit in shared memory")
            _f32vec(norm_w, D, "skinny_chain: norm weight")
            n_out = w.shape[0] // 2 if kind == "swiglu" else w.shape[0]
            if not (out.dtype == torch.bfloat16 and out.shape == (M, n_out) and out.stride(1) == 1
                    and (kind == "store" or w.shape[0] == 2 * n_out)):
                raise KernelError("skinny_chain: out must be bfloat16 [M, N]")
            slot.mode, slot.N = (1 if kind == "swiglu" else 0), n_out
            slot.h_in, slot.norm_w, slot.eps = h.data_ptr(), norm_w.data_ptr(), float(eps)
            slot.w0, slot.K0, slot.scale0 = w.data_ptr(), D, (float(ph[4]) if kind == "swiglu" else 1.0)
            slot.y, slot.ldy = out.data_ptr(), out.stride(0)
        else:
            raise KernelError(f"skinny_chain: unknown phase {kind!r}")
    counter, status = _chain_state(h.device)
    _call("pmm_skinny_chain", ctypes.cast(arr, ctypes.c_void_p), len(phases), M, counter.data_ptr(), status.data_ptr(),
          _stream())


def _tc_status(device: torch.device) -> Tensor:
    return _watch(device).words[0:1]


def tc_gemm_status(device) -> int:
    """0 unless a bounded wait inside a tensor-core kernel gave up (tc_gemm: 1 producer, 2 MMA
    issuer, 3 epilogue; attention_tc: 11..15; skinny_tc: 21..24; decode attention: 31..33).  Reading it waits for the device."""
    return int(_tc_status(torch.device(device)).item())


def _skinny_tc_operand(x: Tensor, w: Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.stride(1) == 1 and w.is_contiguous() and x.shape[1] == w.shape[1] and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def skinny_tc_supported(kind: str, x: Tensor, weight: Tensor, out: Optional[Tensor] = None) -> bool:
    """Whether the tcgen05 weight-streaming product (1..64 tokens) takes these operands; kind is
    "store", "swiglu" (both keep all of K resident: at most 1,024 columns) or "residual"."""
    if not _skinny_tc_operand(x, weight):
        return False
    mode = {"store": 0, "swiglu": 1, "residual": 2}[kind]
    T, K = x.shape
    n = weight.shape[0] // 2 if kind == "swiglu" else weight.shape[0]
    ldy = 8
    if out is not None and kind != "residual":
        if out.dtype != torch.bfloat16 or out.stride(1) != 1 or out.data_ptr() % 16:
            return False
        ldy = out.stride(0)
    return bool(_fn("pmm_skinny_tc_supported")(mode, T, n, K, 0, x.stride(0), 0, ldy))


def skinny_tc_linear(x: Tensor, weight: Tensor, out: Tensor) -> None:
    """out[T, N] (bfloat16) = x @ weight^T for up to 64 tokens on the tcgen05 tensor cores."""
    _cuda(x, weight, out)
    if not (skinny_tc_supported("store", x, weight, out) and out.shape == (x.shape[0], weight.shape[0])):
        raise KernelError("skinny_tc_linear: operands not supported (bfloat16, <= 64 tokens, K <= 1024 and a "
                          "multiple of 8, aligned rows)")
    T, K = x.shape
    _call("pmm_skinny_tc", 0, T, weight.shape[0], x.data_ptr(), x.stride(0), weight.data_ptr(), K, 1.0, None, 0, None, 0,
          0.0, out.data_ptr(), out.stride(0), None, _tc_status(x.device).data_ptr(), _stream())


def skinny_tc_swiglu(x: Tensor, gate_up: Tensor, gate_mult: float, out: Tensor) -> None:
    """out[T, F] = silu(gate * gate_mult) * up with [gate | up] = x @ gate_up^T (tcgen05, up to 64 tokens)."""
    _cuda(x, gate_up, out)
    F = gate_up.shape[0] // 2
    if not (gate_up.shape[0] == 2 * F and skinny_tc_supported("swiglu", x, gate_up, out) and out.shape == (x.shape[0], F)):
        raise KernelError("skinny_tc_swiglu: operands not supported (bfloat16, <= 64 tokens, K <= 1024 and a "
                          "multiple of 8, aligned rows)")
    T, K = x.shape
    _call("pmm_skinny_tc", 1, T, F, x.data_ptr(), x.stride(0), gate_up.data_ptr(), K, float(gate_mult), None, 0, None, 0,
          0.0, out.data_ptr(), out.stride(0), None, _tc_status(x.device).data_ptr(), _stream())


def skinny_tc_residual(h: Tensor, products: Sequence[Tuple[Tensor, Tensor, float]]) -> None:
    """h[T, N] += sum_i scale_i * (x_i @ w_i^T) for one or two products (tcgen05, up to 64 tokens;
    float32 atomics, K in slices of at most 1,024 columns)."""
    if not (1 <= len(products) <= 2):
        raise KernelError("skinny_tc_residual: one or two products")
    _cuda(h)
    T, N = h.shape
    if not (h.dtype == torch.float32 and h.is_contiguous()):
        raise KernelError("skinny_tc_residual: h must be contiguous float32")
    flat = []
    for x, w, sc in products:
        _cuda(x, w)
        if not (skinny_tc_supported("residual", x, w) and x.shape[0] == T and w.shape[0] == N):
            raise KernelError("skinny_tc_residual: operands not supported (bfloat16, <= 64 tokens, K a multiple of "
                              "8, aligned rows)")
        flat.append((x.data_ptr(), x.stride(0), w.data_ptr(), x.shape[1], float(sc)))
    a0 = flat[0]
    a1 = flat[1] if len(flat) > 1 else (None, 0, None, 0, 0.0)
    _call("pmm_skinny_tc", 2, T, N, a0[0], a0[1], a0[2], a0[3], a0[4], a1[0], a1[1], a1[2], a1[3], a1[4], None, 0,
          h.data_ptr(), _tc_status(h.device).data_ptr(), _stream())


def tc_gemm_supported(x: Tensor, weight: Tensor, n_out: int, swiglu: bool) -> bool:
    """Whether the tcgen05 product takes these operands (bfloat16, K a multiple of 64, output
    columns a multiple of 128 for SwiGLU or 256 otherwise, 16-byte aligned rows)."""
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_cuda:
        return False
    if x.dim() != 2 or x.stride(1) != 1 or not weight.is_contiguous() or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return False
    return bool(_fn("pmm_tc_gemm_supported")(1 if swiglu else 0, x.shape[1], n_out, x.stride(0), n_out))


def tc_gemm_swiglu(x: Tensor, gate_up: Tensor, gate_mult: float, out: Tensor) -> None:
    """out[T, F] = silu((x Wg^T) * gate_mult) * (x Wu^T), gate_up = [Wg; Wu]: one tcgen05 kernel
    (TMA operands, accumulator in tensor memory, activation in the epilogue)."""
    _cuda(x, gate_up, out)
    T, K = x.shape
    F = gate_up.shape[0] // 2
    if not (gate_up.shape == (2 * F, K) and out.shape == (T, F) and out.is_contiguous() and out.dtype == torch.bfloat16):
        raise KernelError("tc_gemm_swiglu: out must be contiguous bfloat16 [T, F] for gate_up [2F, K]")
    if not (tc_gemm_supported(x, gate_up, F, True)):
        raise KernelError("tc_gemm_swiglu: sizes or alignment outside what the kernel takes")
    _call("pmm_tc_gemm", 1, x.data_ptr(), x.stride(0), gate_up.data_ptr(), out.data_ptr(), out.stride(0), T, K, F,
          float(gate_mult), _tc_status(x.device).data_ptr(), _stream())


def tc_gemm_gelu_glu(x: Tensor, gate_up: Tensor, gate_mult: float, out: Tensor) -> None:
    """out[T, F] = gelu_tanh((x Wg^T) * gate_mult) * (x Wu^T), gate_up = [Wg; Wu]: the tcgen05 launch of
    `tc_gemm_swiglu` with the tanh form of GELU in its epilogue."""
    _cuda(x, gate_up, out)
    T, K = x.shape
    F = gate_up.shape[0] // 2
    if not (gate_up.shape == (2 * F, K) and out.shape == (T, F) and out.is_contiguous() and out.dtype == torch.bfloat16
            and tc_gemm_supported(x, gate_up, F, True)):
        raise KernelError("tc_gemm_gelu_glu: sizes or alignment outside what the kernel takes")
    _call("pmm_tc_gemm_act", 3, x.data_ptr(), x.stride(0), gate_up.data_ptr(), out.data_ptr(), out.stride(0), T, K, F,
          float(gate_mult), 0.0, 0.0, _tc_status(x.device).data_ptr(), _stream())


def tc_gemm_clamped_glu(x: Tensor, gate_up: Tensor, limit: float, alpha: float, shift: float, out: Tensor) -> None:
    """out[T, F] = g * sigmoid(alpha g) * (u + shift), g = min(x Wg^T, limit), u = clamp(x Wu^T, -limit, limit), with
    gate_up = [Wg; Wu] ([2F, K]): one tcgen05 launch, the activation in its epilogue."""
    _cuda(x, gate_up, out)
    T, Kd = x.shape
    F = out.shape[1]
    if not (gate_up.shape == (2 * F, Kd) and out.shape[0] == T and tc_gemm_supported(x, gate_up, F, True)
            and out.dtype == torch.bfloat16 and out.stride(1) == 1):
        raise KernelError("tc_gemm_clamped_glu: sizes or alignment outside what the kernel takes")
    _call("pmm_tc_gemm_act", 2, x.data_ptr(), x.stride(0), gate_up.data_ptr(), out.data_ptr(), out.stride(0), T, Kd, F,
          float(limit), float(alpha), float(shift), _tc_status(x.device).data_ptr(), _stream())


def tc_gemm(x: Tensor, weight: Tensor, out: Tensor) -> None:
    """out[T, N] = x @ weight^T on tcgen05 (bfloat16 in and out, float accumulation)."""
    _cuda(x, weight, out)
    T, K = x.shape
    N = weight.shape[0]
    if not (weight.shape == (N, K) and out.shape == (T, N) and out.stride(1) == 1 and out.dtype == torch.bfloat16
            and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0):
        raise KernelError("tc_gemm: out must be bfloat16 [T, N], rows 16-byte aligned")
    if not (tc_gemm_supported(x, weight, N, False)):
        raise KernelError("tc_gemm: sizes or alignment outside what the kernel takes")
    _call("pmm_tc_gemm", 0, x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0), T, K, N,
          1.0, _tc_status(x.device).data_ptr(), _stream())


def attention_tc_supported(n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 attention for prompt portions takes this shape (bfloat16, head size 64,
    a group size that divides 128, pages of a multiple of 64 tokens)."""
    return bool(_fn("pmm_attention_tc_supported")(n_q_heads, n_kv_heads, head_dim, page_size))


def attention_tc(q: Tensor, pool: Tensor, block_table: Tensor, positions: Tensor, cu_seqlens: Tensor,
                 new_lens: Sequence[int], out: Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int,
                 softmax_scale: float, window: int = 0, n_splits: int = 1, split_len: int = 0,
                 scratch: Optional[Tensor] = None, split_counter: Optional[Tensor] = None,
                 sink: Optional[Tensor] = None, keep_first: int = 0, lse: Optional[Tensor] = None,
                 seq_of: Optional[Tensor] = None) -> None:
    """Causal attention of prompt portions over the paged cache on the fifth-generation tensor cores
    (TMA tiles straight from the pages, scores and P V in tensor memory, one thread per query row
    for the softmax).  Same contract as paged_attention with rotated queries and a cache that holds
    the step's keys already; 128 rows of (token, query head of a group) per block.  ``keep_first`` > 0 behind a
    window: one key split, ``lse`` scratch and ``seq_of``, as in paged_attention."""
    _cuda(q, pool, block_table, positions, cu_seqlens, out, scratch, split_counter)
    T = q.shape[0]
    keep = int(keep_first) if window > 0 else 0
    if keep > 0 and not (n_splits == 1 and seq_of is not None):
        raise KernelError("attention_tc: kept first keys take one key split and seq_of")
    if not (q.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and q.is_contiguous() and out.is_contiguous() and q.shape == (T, n_q_heads * head_dim) and out.shape == q.shape):
        raise KernelError("attention_tc: q and out must be contiguous bfloat16 [T, Hq*Dh]")
    if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == n_kv_heads * head_dim and pool.is_contiguous()):
        raise KernelError("attention_tc: pool must be contiguous [pages, 2, page_size, Hkv*Dh]")
    if not (attention_tc_supported(n_q_heads, n_kv_heads, head_dim, pool.shape[2])):
        raise KernelError("attention_tc: head size 64 or 128, at most 64 query heads per key/value head and pages "
                          "of a multiple of 64 tokens")
    _i32(block_table, "attention_tc: block_table")
    _i32(positions, "attention_tc: positions")
    _i32(cu_seqlens, "attention_tc: cu_seqlens")
    per_tile = 128 // (n_q_heads // n_kv_heads)
    n_tiles = sum((n + per_tile - 1) // per_tile for n in new_lens)
    part_o = part_ml = counter = None
    if n_splits > 1:
        need = attention_scratch_floats(T, n_q_heads, head_dim, n_splits)
        if not (scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
                and scratch.numel() >= need and scratch.data_ptr() % 16 == 0):
            raise KernelError(f"attention_tc: split keys need {need} floats of scratch")
        if not (split_len > 0 and split_len % 64 == 0 and n_splits <= 64):
            raise KernelError("attention_tc: split_len must be a multiple of 64")
        if not (split_counter is not None and split_counter.numel() >= n_tiles * n_kv_heads):
            raise KernelError("attention_tc: split keys need a counter per (row tile, key/value head)")
        _i32(split_counter, "attention_tc: split_counter")
        part_o = scratch.data_ptr()
        part_ml = part_o + 4 * T * n_q_heads * n_splits * head_dim
        counter = split_counter.data_ptr()
    _call("pmm_attention_tc", q.data_ptr(), pool.data_ptr(), pool.shape[0], block_table.data_ptr(), block_table.shape[1],
          positions.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(), part_o, part_ml, float(softmax_scale), int(window),
          int(split_len), int(n_splits), pool.shape[2], len(new_lens), n_tiles, n_q_heads, n_kv_heads, head_dim, counter,
          _tc_status(q.device).data_ptr(), _ptr(sink), _lse_ptr(lse, T, n_q_heads) if keep > 0 else None, _stream())
    if keep > 0:
        kept_first_merge(q, pool, block_table, positions, seq_of, out, lse, n_q_heads, n_kv_heads, head_dim, softmax_scale,
                         window, keep)


def silu_mul(gate_up: Tensor, gate_mult: float, out: Tensor) -> None:
    """out[t, f] = silu(gate_up[t, f] * gate_mult) * gate_up[t, F + f]."""
    _cuda(gate_up, out)
    ld = _rows_view(gate_up, "silu_mul: gate_up")
    T, F2 = gate_up.shape
    if not (F2 % 2 == 0 and out.shape == (T, F2 // 2) and out.is_contiguous() and out.dtype == gate_up.dtype):
        raise KernelError("silu_mul: out must be contiguous [T, F] for gate_up [T, 2F]")
    _call("pmm_silu_mul", gate_up.data_ptr(), ld, float(gate_mult), out.data_ptr(), T, F2 // 2,
          _dt(gate_up), _stream())


def gelu_tanh_mul(gate_up: Tensor, gate_mult: float, out: Tensor) -> None:
    """out[t, f] = gelu_tanh(gate_up[t, f] * gate_mult) * gate_up[t, F + f], gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi)
    (z + 0.044715 z^3)))."""
    _cuda(gate_up, out)
    ld = _rows_view(gate_up, "gelu_tanh_mul: gate_up")
    T, F2 = gate_up.shape
    if not (F2 % 2 == 0 and out.shape == (T, F2 // 2) and out.is_contiguous() and out.dtype == gate_up.dtype):
        raise KernelError("gelu_tanh_mul: out must be contiguous [T, F] for gate_up [T, 2F]")
    _call("pmm_gelu_tanh_mul", gate_up.data_ptr(), ld, float(gate_mult), out.data_ptr(), T, F2 // 2, _dt(gate_up), _stream())


def sigmoid_gate(a: Tensor, g: Tensor, scale: float, out: Tensor, n_heads: int, stored_dim: int, dim: int) -> None:
    """out[t, h*dim + i] = scale * a[t, h*stored_dim + i] * sigmoid(g[t, h*dim + i]) for i < dim."""
    _cuda(a, g, out)
    T = a.shape[0]
    if not (a.shape == (T, n_heads * stored_dim) and g.shape == (T, n_heads * dim) and out.shape == (T, n_heads * dim)
            and a.dtype == g.dtype == out.dtype and stored_dim >= dim):
        raise KernelError("sigmoid_gate: a [T, H*stored], g and out [T, H*dim] of one type")
    ld_a, ld_g, ld_o = (_rows_view(t, "sigmoid_gate") for t in (a, g, out))
    _call("pmm_sigmoid_gate", a.data_ptr(), ld_a, g.data_ptr(), ld_g, float(scale), out.data_ptr(), ld_o, T, n_heads,
          stored_dim, dim, _dt(a), _stream())


def clamped_glu(gate_up: Tensor, limit: float, alpha: float, shift: float, out: Tensor) -> None:
    """out = g * sigmoid(alpha g) * (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit),
    [gate | up] = gate_up [T, 2F]."""
    _cuda(gate_up, out)
    T, F2 = gate_up.shape
    if not (F2 % 2 == 0 and out.shape == (T, F2 // 2) and out.is_contiguous() and out.dtype == gate_up.dtype):
        raise KernelError("clamped_glu: gate_up [T, 2F], out contiguous [T, F] of the same type")
    _call("pmm_clamped_glu", gate_up.data_ptr(), _rows_view(gate_up, "clamped_glu"), float(limit), float(alpha),
          float(shift), out.data_ptr(), T, F2 // 2, _dt(out), _stream())


# ----------------------------------------------------------------------------- latent attention
def latent_padded_dim(kv_rank: int, rot_dim: int) -> int:
    """The head size the attention kernels see for a latent of ``kv_rank`` entries and a rotated key part of
    ``rot_dim``: the next of 16, 32, 64, 128 (the sizes the tensor-core kernels take), beyond that a multiple of 16."""
    need = kv_rank + rot_dim
    for d in (16, 32, 64, 128):
        if need <= d:
            return d
    return (need + 15) // 16 * 16


def latent_norm_store(q_lat: Tensor, kv_lat: Tensor, q_w: Tensor, kv_w: Tensor, eps: float, inv_freq: Optional[Tensor],
                      positions: Tensor, seq_of: Tensor, block_table: Tensor, pool: Tensor, cq: Tensor, kv_rank: int,
                      rot_dim: int, rot_dims: int, half_layout: bool = False, queries: Optional[Tuple] = None) -> None:
    """cq = rms(q_lat) * q_w; the cache rows of the step's tokens: key row [rms(kv_lat[:kv_rank]) * kv_w | the last
    rot_dim entries of kv_lat, of which the first rot_dims turn in neighbouring pairs | 0], value row [the normed
    latent | 0], into ``pool`` [pages, 2, page_size, Dp].  Norms, angles, sines and cosines are float.
    ``half_layout``: entries (i, i + rot_dims/2) turn together instead of neighbours.  ``q_lat`` None (with q_w and
    cq None): the queries have no latent, only the cache rows are made.  ``queries`` = (q [T, heads * (dim +
    rot_dim)], q_out [T, heads * Dp], heads, dim): `latent_query_rot`'s work for these queries in the same launch."""
    _cuda(q_lat, kv_lat, q_w, kv_w, inv_freq, positions, seq_of, block_table, pool, cq)
    T = kv_lat.shape[0]
    if q_lat is None:
        if not (q_w is None and cq is None):
            raise KernelError("latent_norm_store: no query latent means no q_w and no cq")
        q_rank = 0
        if not (kv_lat.shape == (T, kv_rank + rot_dim) and kv_lat.dtype == pool.dtype and kv_lat.stride(1) == 1):
            raise KernelError("latent_norm_store: kv_lat [T, kv_rank + rot_dim] of the pool's type")
    else:
        q_rank = q_lat.shape[1]
        if not (q_lat.shape[0] == T and kv_lat.shape == (T, kv_rank + rot_dim)
                and q_lat.dtype == kv_lat.dtype == pool.dtype == cq.dtype and q_lat.stride(1) == 1 and kv_lat.stride(1) == 1):
            raise KernelError("latent_norm_store: q_lat [T, q_rank], kv_lat [T, kv_rank + rot_dim] of the pool's type")
        if not (cq.shape == (T, q_rank) and cq.is_contiguous()):
            raise KernelError("latent_norm_store: cq must be contiguous [T, q_rank]")
    if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.is_contiguous() and pool.shape[3] >= kv_rank + rot_dim):
        raise KernelError("latent_norm_store: pool must be contiguous [pages, 2, page_size, Dp >= kv_rank + rot_dim]")
    if q_lat is not None:
        _f32vec(q_w, q_rank, "latent_norm_store: q_w")
    _f32vec(kv_w, kv_rank, "latent_norm_store: kv_w")
    _f32vec(inv_freq, rot_dims // 2, "latent_norm_store: inv_freq")
    _i32(positions, "latent_norm_store: positions")
    _i32(seq_of, "latent_norm_store: seq_of")
    _i32(block_table, "latent_norm_store: block_table")
    _call("pmm_latent_norm_store", _ptr(q_lat), q_lat.stride(0) if q_lat is not None else 0, kv_lat.data_ptr(),
          kv_lat.stride(0), _ptr(q_w), kv_w.data_ptr(), float(eps), _ptr(inv_freq), positions.data_ptr(), seq_of.data_ptr(),
          block_table.data_ptr(), block_table.shape[1], pool.data_ptr(), pool.shape[2], _ptr(cq), T, q_rank, int(kv_rank),
          int(rot_dim), int(rot_dims), pool.shape[3], int(bool(half_layout)), *_latent_queries(queries, T, rot_dim, pool),
          _dt(kv_lat), _stream())


def _latent_queries(queries: Optional[Tuple], T: int, rot_dim: int, pool: Tensor):
    if queries is None:
        return None, 0, None, 0, 0
    q, q_out, heads, dim = queries
    _cuda(q, q_out)
    if not (q.shape == (T, heads * (dim + rot_dim)) and q.stride(1) == 1 and q.dtype == q_out.dtype == pool.dtype
            and q_out.shape == (T, heads * pool.shape[3]) and q_out.is_contiguous()):
        raise KernelError("latent_norm_store: queries [T, H * (dim + rot_dim)], q_out contiguous [T, H * Dp] of the pool's type")
    return q.data_ptr(), q.stride(0), q_out.data_ptr(), int(heads), int(dim)


def latent_query_rot(q: Tensor, inv_freq: Optional[Tensor], positions: Tensor, q_out: Tensor, heads: int, dim: int,
                     rot_dim: int, rot_dims: int, kv_rank: int, padded_dim: int, half_layout: bool = False) -> None:
    """q [T, heads * (dim + rot_dim)]: the rotated part of every head turns and goes to q_out[t, h, kv_rank ..
    kv_rank + rot_dim); the entries from there to padded_dim become zero; the first kv_rank stay as they are."""
    _cuda(q, inv_freq, positions, q_out)
    T = q.shape[0]
    if not (q.shape[1] == heads * (dim + rot_dim) and q.stride(1) == 1 and q.dtype == q_out.dtype
            and q_out.shape == (T, heads * padded_dim) and q_out.is_contiguous()):
        raise KernelError("latent_query_rot: q [T, H * (dim + rot_dim)], q_out contiguous [T, H * Dp] of one type")
    _f32vec(inv_freq, rot_dims // 2, "latent_query_rot: inv_freq")
    _i32(positions, "latent_query_rot: positions")
    _call("pmm_latent_query_rot", q.data_ptr(), q.stride(0), _ptr(inv_freq), positions.data_ptr(), q_out.data_ptr(), T,
          int(heads), int(dim), int(rot_dim), int(rot_dims), int(kv_rank), int(padded_dim), int(bool(half_layout)), _dt(q),
          _stream())


def head_gate(a: Tensor, g: Optional[Tensor], scale: float, out: Tensor, heads: int, vdim: int) -> None:
    """out[t, h * vdim + i] = scale * a[t, h * vdim + i] * sigmoid(g[t, h]) (g None: scale only)."""
    _cuda(a, g, out)
    T = a.shape[0]
    if not (a.shape == (T, heads * vdim) and out.shape == a.shape and a.stride(1) == 1 and out.stride(1) == 1
            and a.dtype == out.dtype):
        raise KernelError("head_gate: a and out [T, H * vdim] of one type")
    if g is not None and not (g.shape == (T, heads) and g.stride(1) == 1 and g.dtype == a.dtype):
        raise KernelError("head_gate: g [T, H] of a's type")
    _call("pmm_head_gate", a.data_ptr(), a.stride(0), _ptr(g), g.stride(0) if g is not None else 0, float(scale),
          out.data_ptr(), out.stride(0), T, int(heads), int(vdim), _dt(a), _stream())


def head_linear(x: Tensor, w: Tensor, out: Tensor) -> None:
    """out[t, h, :] = x[t, h, :] @ w[h]: a product per head, x [T, H, K] and out [T, H, N] views with unit inner
    stride, w [H, K, N] (any strides the library takes).  Float32 operands stay true float32."""
    _cuda(x, w, out)
    H = w.shape[0]
    if not (x.dim() == 3 and out.dim() == 3 and x.shape[1] == H and out.shape[1] == H and x.shape[2] == w.shape[1]
            and out.shape[2] == w.shape[2] and x.shape[0] == out.shape[0] and x.stride(2) == 1 and out.stride(2) == 1
            and x.dtype == w.dtype == out.dtype):
        raise KernelError("head_linear: x [T, H, K], w [H, K, N], out [T, H, N] of one type")
    if x.shape[0] == 0:
        return
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        torch.bmm(x.transpose(0, 1), w, out=out.transpose(0, 1))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


# ----------------------------------------------------------------------------- updates of the residual stream
def token_gated_update_fits(width: int, rank: int) -> bool:
    return bool(_fn("pmm_token_gated_update_fits")(int(width), int(rank)))


def token_gated_update(h: Tensor, branches: Sequence[Tuple[Tensor, float]], tokens: Tensor, table: Tensor, col0: int,
                       w_gate: Tensor, w_proj_t: Tensor, norm_w: Tensor, eps: float,
                       w_proj_rows: Optional[Tensor] = None) -> None:
    """h <- x + rms(Wp (gelu_tanh(Wg x) * e)) * norm_w with x = h + sum(scale_i * branch_i) (at most two branches)
    and e = table[token, col0 : col0 + R]; h [T, D] float32 in place, Wg [R, D], Wp given transposed: Wp^T [R, D]
    (its rows are then read side by side).  With ``w_proj_rows`` (Wp [D, R] as stored) bfloat16 steps of many
    tokens run on the tensor cores where the sizes allow: x and g enter the two products rounded to bfloat16
    there, sums, activation, root mean square and the stream stay float."""
    items = list(branches)
    w_proj = w_proj_t
    if w_proj_rows is not None:
        _cuda(w_proj_rows)
        if not (w_proj_rows.shape == (w_proj_t.shape[1], w_proj_t.shape[0]) and w_proj_rows.is_contiguous()
                and w_proj_rows.dtype == w_proj_t.dtype):
            raise KernelError("token_gated_update: w_proj_rows must be contiguous [D, R] of the matrices' type")
    _cuda(h, tokens, table, w_gate, w_proj, norm_w, *[b for b, _ in items])
    T, D = h.shape
    R = w_gate.shape[0]
    if not (h.dtype == torch.float32 and h.is_contiguous() and len(items) <= 2):
        raise KernelError("token_gated_update: h contiguous float32 and at most two branches")
    if not (w_gate.shape == (R, D) and w_proj.shape == (R, D) and w_gate.is_contiguous() and w_proj.is_contiguous()
            and w_gate.dtype == w_proj.dtype == table.dtype and table.dim() == 2 and table.stride(1) == 1
            and 0 <= col0 and col0 + R <= table.shape[1]):
        raise KernelError("token_gated_update: Wg [R, D], Wp^T [R, D] and the table of one type, the columns inside it")
    for b, _ in items:
        if not (b.shape == h.shape and b.is_contiguous() and b.dtype == w_gate.dtype):
            raise KernelError("token_gated_update: branches contiguous [T, D] of the matrices' type")
    if not token_gated_update_fits(D, R):
        raise KernelError("token_gated_update: a token's rows do not fit the shared memory")
    _f32vec(norm_w, D, "token_gated_update: norm_w")
    _i32(tokens, "token_gated_update: tokens")
    (a, sa), (b, sb) = (items + [(None, 0.0), (None, 0.0)])[:2]
    _call("pmm_token_gated_update", h.data_ptr(), _ptr(a), float(sa), _ptr(b), float(sb), tokens.data_ptr(), table.data_ptr(),
          table.stride(0), int(col0), w_gate.data_ptr(), w_proj.data_ptr(), _ptr(w_proj_rows), norm_w.data_ptr(), float(eps), T, D, R,
          _dt(w_gate), _stream())


def cast_rows(h: Tensor, branches: Sequence[Tuple[Tensor, float]], out: Tensor) -> None:
    """h <- h + sum(scale_i * branch_i) (at most two), out[t, :D] = h[t] in out's type (out may be a column block)."""
    items = list(branches)
    _cuda(h, out, *[b for b, _ in items])
    T, D = h.shape
    if not (h.dtype == torch.float32 and h.is_contiguous() and out.shape == (T, D) and out.stride(1) == 1 and len(items) <= 2):
        raise KernelError("cast_rows: h contiguous float32 [T, D], out [T, D] with unit inner stride, at most two branches")
    for b, _ in items:
        if not (b.shape == h.shape and b.is_contiguous() and b.dtype == out.dtype):
            raise KernelError("cast_rows: branches contiguous [T, D] of out's type")
    (a, sa), (b, sb) = (items + [(None, 0.0), (None, 0.0)])[:2]
    _call("pmm_cast_rows", h.data_ptr(), _ptr(a), float(sa), _ptr(b), float(sb), out.data_ptr(), out.stride(0), T, D,
          _dt(out), _stream())


def relu_squared(x: Tensor, out: Tensor) -> None:
    """out = max(x, 0)^2, element-wise over [T, F] (rows may be strided)."""
    _cuda(x, out)
    if not (x.dim() == 2 and out.shape == x.shape and x.stride(1) == 1 and out.stride(1) == 1 and x.dtype == out.dtype):
        raise KernelError("relu_squared: x and out [T, F] of one type with unit inner stride")
    _call("pmm_relu_squared", x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), x.shape[0], x.shape[1], _dt(x),
          _stream())


# ----------------------------------------------------------------------------- routed feed-forward
def moe_route(x: Tensor, router_w: Tensor, router_b: Optional[Tensor], top: int, ids: Tensor, weights: Tensor,
              scored = False, correction: Optional[Tensor] = None, groups: int = 1, keep: int = 1,
              scale: float = 1.0, gate_w: Optional[Tensor] = None, gate_out: Optional[Tensor] = None) -> None:
    """ids, weights [T, top] of z = x Wr^T + br (float arithmetic).  Plain: the ``top`` largest z and their softmax.
    ``scored``: s = sigmoid(z); the ``top`` largest of s + correction among the experts of the ``keep`` groups (of
    ``groups`` equal groups of neighbours) whose two largest s + correction sum highest; weights the chosen s over
    their sum, times ``scale``.  ``scored`` "softmax": s = softmax(z) over all experts, a group counts by its largest
    s + correction, and the weights are the chosen s times ``scale`` (not divided by their sum).  ``gate_w`` [D] float32: gate_out[t] = sigmoid(x[t] . gate_w) as well."""
    _cuda(x, router_w, router_b, ids, weights, correction, gate_w, gate_out)
    T, D = x.shape
    E = router_w.shape[0]
    if not (router_w.shape == (E, D) and router_w.dtype == torch.float32 and router_w.is_contiguous()):
        raise KernelError("moe_route: router weight [E, D] float32")
    if router_b is not None:
        _f32vec(router_b, E, "moe_route: router bias")
    _f32vec(correction, E, "moe_route: correction")
    if not (ids.shape == (T, top) and ids.dtype == torch.int32 and ids.is_contiguous() and weights.shape == (T, top)
            and weights.dtype == torch.float32 and weights.is_contiguous() and 1 <= top <= E):
        raise KernelError("moe_route: ids int32 and weights float32, both contiguous [T, top], top <= experts")
    if scored and not (groups >= 1 and E % groups == 0 and 1 <= keep <= groups and top <= keep * (E // groups)):
        raise KernelError("moe_route: groups must divide the experts, keep <= groups, top <= keep * experts / groups")
    if gate_w is not None:
        _f32vec(gate_w, D, "moe_route: gate_w")
        if not (gate_out is not None and gate_out.dtype == torch.float32 and gate_out.is_contiguous() and gate_out.numel() == T):
            raise KernelError("moe_route: gate_out must be contiguous float32 [T]")
    _call("pmm_moe_route", x.data_ptr(), _rows_view(x, "moe_route"), router_w.data_ptr(), _ptr(router_b), ids.data_ptr(),
          weights.data_ptr(), T, D, E, int(top), 2 if scored == "softmax" else int(bool(scored)), _ptr(correction), int(groups), int(keep), float(scale),
          _ptr(gate_w), _ptr(gate_out) if gate_w is not None else None, _dt(x), _stream())


_MOE_FORMS = {"float": 0, "mma": 1, "mma_few": 2}


def moe_tile_rows(form: str) -> int:
    """Rows of a row tile of the grouped products: ``form`` "float" (CUDA cores, any sizes), "mma" (mma.sync),
    "mma_few" (mma.sync, steps of few pairs) or "tcgen05"."""
    if form == "tcgen05":
        return int(_fn("pmm_moe_tc_tile_rows")())
    return int(_fn("pmm_moe_tile_rows")(_MOE_FORMS[form]))


def moe_plan(ids: Tensor, n_experts: int, form: str, offsets: Tensor, tile_start: Tensor, perm: Tensor) -> None:
    """Sorts the pairs by expert: offsets, tile_start [E + 1] int32 (row tiles of the given form of the grouped
    products), perm [T * top] int32."""
    _cuda(ids, offsets, tile_start, perm)
    A = ids.numel()
    for t, n, what in ((offsets, n_experts + 1, "offsets"), (tile_start, n_experts + 1, "tile_start"), (perm, A, "perm")):
        if not (t.dtype == torch.int32 and t.is_contiguous() and t.numel() == n):
            raise KernelError(f"moe_plan: {what} must be contiguous int32 of {n}")
    _i32(ids, "moe_plan: ids")
    _call("pmm_moe_plan", ids.data_ptr(), A, int(n_experts), moe_tile_rows(form), offsets.data_ptr(),
          tile_start.data_ptr(), perm.data_ptr(), _stream())
    if A > 512:
        global launch_count
        launch_count += 1  # two launches for many pairs


def moe_tc_supported(a: Tensor, w: Tensor, n_out: int) -> bool:
    """Whether the tcgen05 grouped product takes these operands (bfloat16, K a multiple of 64, N of 8)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.stride(1) == 1 and a.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and bool(_fn("pmm_moe_tc_supported")(a.shape[1], int(n_out), a.stride(0))))


def moe_gather_rows(x: Tensor, perm: Tensor, top: int, out: Tensor) -> None:
    """out[i] = x[perm[i] // top]: the token rows in the order of the sorted pairs (bfloat16)."""
    _cuda(x, perm, out)
    A, Kd = out.shape
    if not (x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.is_contiguous() and x.shape[1] == Kd
            and perm.numel() == A and Kd % 8 == 0):
        raise KernelError("moe_gather_rows: bfloat16 rows of a multiple of 8 elements, one output row per pair")
    _call("pmm_moe_gather_rows", x.data_ptr(), _rows_view(x, "moe_gather_rows"), perm.data_ptr(), A, int(top),
          out.data_ptr(), Kd, _stream())


def moe_tc_gemm(a: Tensor, w: Tensor, perm: Tensor, offsets: Tensor, tile_start: Tensor, up: bool, out: Tensor,
                limit: float = 0.0, alpha: float = 0.0, shift: float = 0.0, ungated: bool = False) -> None:
    """The grouped product on the fifth-generation tensor cores.  a [pairs, K]: rows in the order of the sorted
    pairs (the gathered token rows, or the activation); w [E, N (2N), K]; the plan made for "tcgen05" row tiles.
    ``up``: out = act [pairs, N] with the clamped gated activation; else out = y [pairs, N] in the order of the
    pairs (both bfloat16).  ``up`` and ``ungated``: w [E, N, K], out = act [pairs, N] = max(a W^T, 0)^2."""
    _cuda(a, w, perm, offsets, tile_start, out)
    A, Kd = a.shape
    E, N = w.shape[0], out.shape[1]
    if ungated and not up:
        raise KernelError("moe_tc_gemm: only an up product is gated or ungated")
    if not (w.dim() == 3 and w.is_contiguous() and w.shape == (E, (2 if up and not ungated else 1) * N, Kd) and perm.numel() == A
            and out.shape == (A, N) and out.is_contiguous() and out.dtype == torch.bfloat16
            and offsets.numel() == E + 1 and tile_start.numel() == E + 1 and moe_tc_supported(a, w, N)):
        raise KernelError("moe_tc_gemm: operands outside what the kernel takes")
    _call("pmm_moe_tc_gemm", a.data_ptr(), a.stride(0), w.data_ptr(), perm.data_ptr(), offsets.data_ptr(),
          tile_start.data_ptr(), A, E, Kd, N, (2 if ungated else 1) if up else 0, float(limit), float(alpha), float(shift),
          out.data_ptr(), _tc_status(a.device).data_ptr(), _stream())


def moe_gemm_tc_ok(a: Tensor, w: Tensor) -> bool:
    """Whether the grouped product of these operands can run on the tensor cores."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(1) == 1
            and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def moe_gemm(a: Tensor, w: Tensor, perm: Tensor, offsets: Tensor, tile_start: Tensor, top: int, up: bool, out: Tensor,
             form: str, limit: float = 0.0, alpha: float = 0.0, shift: float = 0.0, ungated: bool = False) -> None:
    """Grouped product over the rows of a plan.  ``up``: a = x [T, K], w [E, 2N, K] ([gate | up] rows of
    every expert), out = act [T*top, N] in the storage type, with the clamped gated activation.  Else:
    a = act [T*top, K], w [E, N, K], out = y [T*top, N] in the order of the pairs.  ``up`` and ``ungated``: w [E, N, K],
    out = act [T*top, N] = max(x W^T, 0)^2."""
    _cuda(a, w, perm, offsets, tile_start, out)
    A = perm.numel()
    E = w.shape[0]
    K = a.shape[1]
    N = out.shape[1]
    if ungated and not up:
        raise KernelError("moe_gemm: only an up product is gated or ungated")
    if not (w.dim() == 3 and w.is_contiguous() and w.shape == (E, (2 if up and not ungated else 1) * N, K) and w.dtype == a.dtype):
        raise KernelError("moe_gemm: w must be contiguous [E, N (2N for the gate and up rows), K] of a's type")
    if not (out.shape == (A, N) and out.is_contiguous() and out.dtype == a.dtype):
        raise KernelError("moe_gemm: out [pairs, N] of the operands' type")
    if not (a.shape[0] == (A // top if up else A) and offsets.numel() == E + 1 and tile_start.numel() == E + 1):
        raise KernelError("moe_gemm: rows of a, offsets or tile_start do not fit the plan")
    tensor_cores = _MOE_FORMS[form]  # the plan must have been made for the same form
    if tensor_cores and not moe_gemm_tc_ok(a, w):
        raise KernelError("moe_gemm: the tensor-core forms need bfloat16, K a multiple of 8 and 16-byte aligned rows")
    _call("pmm_moe_gemm", a.data_ptr(), _rows_view(a, "moe_gemm"), w.data_ptr(), perm.data_ptr(), offsets.data_ptr(),
          tile_start.data_ptr(), A, E, int(top), K, N, (2 if ungated else 1) if up else 0, float(limit), float(alpha),
          float(shift), out.data_ptr(), tensor_cores, _dt(a), _stream())


def moe_combine(y: Tensor, weights: Tensor, shared: Optional[Tensor], out: Tensor,
                shared_gate: Optional[Tensor] = None) -> None:
    """out[t] = sum_j weights[t, j] * y[t*top + j] (+ shared[t], times shared_gate[t] where given)."""
    _cuda(y, weights, shared, out, shared_gate)
    T, top = weights.shape
    D = out.shape[1]
    if not (y.shape == (T * top, D) and y.dtype == out.dtype and y.is_contiguous() and out.shape == (T, D)
            and out.is_contiguous() and weights.dtype == torch.float32 and weights.is_contiguous()):
        raise KernelError("moe_combine: y [T*top, D] of out's type, weights [T, top] float32, out contiguous [T, D]")
    if shared is not None and not (shared.shape == (T, D) and shared.is_contiguous() and shared.dtype == out.dtype):
        raise KernelError("moe_combine: shared must be contiguous [T, D] of out's type")
    if shared_gate is not None and not (shared is not None and shared_gate.dtype == torch.float32
                                        and shared_gate.is_contiguous() and shared_gate.numel() == T):
        raise KernelError("moe_combine: shared_gate must be contiguous float32 [T] beside a shared output")
    _call("pmm_moe_combine", y.data_ptr(), weights.data_ptr(), _ptr(shared), _ptr(shared_gate), out.data_ptr(), T, D, top,
          _dt(out), _stream())


def add_row_bias_(x: Tensor, bias: Tensor) -> None:
    """x[t, :] += bias (float32 vector) for a contiguous [T, D] activation."""
    _cuda(x, bias)
    if not (x.dim() == 2 and x.is_contiguous()):
        raise KernelError("add_row_bias_: x must be contiguous [T, D]")
    _f32vec(bias, x.shape[1], "add_row_bias_: bias")
    _call("pmm_add_row_bias", x.data_ptr(), bias.data_ptr(), x.shape[0], x.shape[1], _dt(x), _stream())


_SAMPLE_SCRATCH: Dict[torch.device, Tuple[Tensor, Tensor]] = {}


def ensure_sample_scratch(device, rows: int = 4096) -> Tuple[Tensor, Tensor]:
    """A 64-bit slot and a ticket per row for the blocks that share a row of sample_rows: one pair of
    buffers per device, zero when made and left zero by every launch (launches that use them are
    expected on one stream at a time).  Call it before a step is recorded into a CUDA graph:
    memory cannot be taken for it while a recording is under way."""
    device = torch.device(device)
    have = _SAMPLE_SCRATCH.get(device)
    if have is None or have[0].numel() < rows:
        if not (not torch.cuda.is_current_stream_capturing()):
            raise KernelError("sample_rows: its scratch must exist before a CUDA graph is recorded "
                              "(ensure_sample_scratch)")
        n = max(4096, rows)
        have = (torch.zeros(n, dtype=torch.int64, device=device), torch.zeros(n, dtype=torch.int32, device=device))
        _SAMPLE_SCRATCH[device] = have
    return have


def sample_rows(logits: Tensor, temperature: Optional[Tensor], seeds: Optional[Tensor],
                steps: Optional[Tensor], out: Tensor) -> None:
    """out[r] = argmax (first index on ties) where temperature[r] <= 0, else a draw from
    softmax(logits[r] / temperature[r]) keyed by (seeds[r], steps[r])."""
    _cuda(logits, temperature, seeds, steps, out)
    ld = _rows_view(logits, "sample: logits")
    n, V = logits.shape
    if not (logits.dtype == torch.float32):
        raise KernelError("sample: logits must be float32")
    _i32(out, "sample: out")
    if not (out.numel() == n):
        raise KernelError("sample: one output per row")
    if temperature is not None:
        _f32vec(temperature, n, "sample: temperature")
        if not (seeds is not None and seeds.dtype == torch.int64 and seeds.numel() == n and seeds.is_contiguous()):
            raise KernelError("sample: seeds must be int64 [rows]")
        if not (steps is not None and steps.numel() == n):
            raise KernelError("sample: steps must be int32 [rows]")
        _i32(steps, "sample: steps")
    slots, tickets = ensure_sample_scratch(logits.device, n)
    _call("pmm_sample_rows", logits.data_ptr(), ld, _ptr(temperature), _ptr(seeds), _ptr(steps),
          out.data_ptr(), n, V, slots.data_ptr(), tickets.data_ptr(), _stream())


def l2_prefetch(tensors: Sequence[Tensor]) -> None:
    """Asks the memory system to bring these tensors (contiguous, at most 8 per call, further
    ones in further launches) into L2; nothing waits for it."""
    ts = [t for t in tensors if t is not None and t.numel() > 0]
    for i in range(0, len(ts), 8):
        part = ts[i:i + 8]
        _cuda(*part)
        for t in part:
            if not (t.is_contiguous() and t.data_ptr() % 16 == 0):
                raise KernelError("l2_prefetch: tensors must be contiguous and 16-byte aligned")
        ptrs = (ctypes.c_void_p * len(part))(*[t.data_ptr() for t in part])
        sizes = (ctypes.c_longlong * len(part))(*[t.numel() * t.element_size() for t in part])
        _call("pmm_l2_prefetch", ctypes.cast(ptrs, ctypes.c_void_p), ctypes.cast(sizes, ctypes.c_void_p), len(part),
              _stream())


# ----------------------------------------------------------------------------- residual lanes, normed sums
HC_MAX_LANES = 8


def hc_mix_norm(lanes_in: Tensor, lanes_out: Optional[Tensor], y: Optional[Tensor], mix: Optional[Tensor],
                out_w: Optional[Tensor], in_w: Optional[Tensor], norm_w: Optional[Tensor], eps: float,
                normed: Optional[Tensor], rows: Optional[Tensor] = None) -> None:
    """Residual state in n lanes [n, T, D] (float32).  Folds a sublayer's result y into the lanes,
    x_t <- sum_s mix[s, t] x_s + out_w[t] y (when y is given), writes them to ``lanes_out`` (may be
    ``lanes_in``; not written with ``rows``), and writes normed = rmsnorm(sum_s in_w[s] x_s) * norm_w
    (when asked for; of the listed rows only, with ``rows``).  ``lanes_in`` may be one [T, D] that every
    lane starts from (expanded without a copy: lane stride 0)."""
    _cuda(lanes_in, lanes_out, y, mix, out_w, in_w, norm_w, normed, rows)
    if lanes_out is not None:
        n, T, D = lanes_out.shape
    else:
        n, T, D = lanes_in.shape
    if not (lanes_in.dtype == torch.float32 and lanes_in.shape == (n, T, D) and lanes_in.stride(2) == 1
            and lanes_in.stride(1) == D and 1 <= n <= HC_MAX_LANES):
        raise KernelError("hc_mix_norm: lanes must be float32 [n <= 8, T, D] with contiguous rows")
    if lanes_out is not None and not (lanes_out.dtype == torch.float32 and lanes_out.is_contiguous()):
        raise KernelError("hc_mix_norm: lanes_out must be contiguous float32 [n, T, D]")
    y_dt = 0
    if y is not None:
        if not (y.shape == (T, D) and y.is_contiguous()):
            raise KernelError("hc_mix_norm: y must be contiguous [T, D]")
        _f32vec(mix, n * n, "hc_mix_norm: mix")
        _f32vec(out_w, n, "hc_mix_norm: out_w")
        y_dt = _dt(y)
    R = T
    if rows is not None:
        _i32(rows, "hc_mix_norm: rows")
        R = rows.numel()
    dt = 0
    if normed is not None:
        _f32vec(in_w, n, "hc_mix_norm: in_w")
        _f32vec(norm_w, D, "hc_mix_norm: norm_w")
        if not (normed.shape == (R, D) and normed.is_contiguous()):
            raise KernelError("hc_mix_norm: normed must be contiguous [rows, D]")
        if D * 4 > 200 * 1024:
            raise KernelError(f"hc_mix_norm: width {D} exceeds one block's shared memory")
        dt = _dt(normed)
    _call("pmm_hc_mix_norm", lanes_in.data_ptr(), lanes_in.stride(0), _ptr(lanes_out),
          lanes_out.stride(0) if lanes_out is not None else 0, n, _ptr(y), _ptr(mix), _ptr(out_w), _ptr(in_w),
          _ptr(norm_w), float(eps), _ptr(normed), _ptr(rows), R, D, dt, y_dt, _stream())


def normed_sum(branches: Sequence[Tuple[Tensor, Tensor]], eps: float, scale: float, out: Tensor,
               biases: Optional[Sequence[Optional[Tensor]]] = None) -> None:
    """out = scale * sum_b rmsnorm(x_b + bias_b) * w_b over up to four (x_b [T, D], w_b [D] float32); out
    is float32 or of the branches' type.  ``biases``: per branch a float32 [D] (or None) added to the
    branch before its norm (a projection's bias that no launch of its own has to add)."""
    xs = [b[0] for b in branches]
    _cuda(out, *xs, *[b[1] for b in branches])
    T, D = out.shape
    if not (1 <= len(branches) <= 4 and out.is_contiguous()):
        raise KernelError("normed_sum: one to four branches, contiguous out")
    for x, w in branches:
        if not (x.shape == (T, D) and x.dtype == xs[0].dtype):
            raise KernelError("normed_sum: branches must be [T, D] of one type")
        _rows_view(x, "normed_sum: branch")
        _f32vec(w, D, "normed_sum: weight")
    if not (out.dtype in (torch.float32, xs[0].dtype)):
        raise KernelError("normed_sum: out must be float32 or of the branches' type")
    n = len(branches)
    ptrs = (ctypes.c_void_p * n)(*[x.data_ptr() for x in xs])
    lds = (ctypes.c_longlong * n)(*[x.stride(0) for x in xs])
    ws = (ctypes.c_void_p * n)(*[w.data_ptr() for _, w in branches])
    bs = None
    if biases is not None and any(b is not None for b in biases):
        if len(biases) != n:
            raise KernelError("normed_sum: one bias (or None) per branch")
        for b in biases:
            _cuda(b)
            _f32vec(b, D, "normed_sum: bias")
        bs = ctypes.cast((ctypes.c_void_p * n)(*[b.data_ptr() if b is not None else None for b in biases]), ctypes.c_void_p)
    _call("pmm_normed_sum", ctypes.cast(ptrs, ctypes.c_void_p), ctypes.cast(lds, ctypes.c_void_p),
          ctypes.cast(ws, ctypes.c_void_p), bs, n, float(eps), float(scale), out.data_ptr(),
          int(out.dtype == torch.float32 and xs[0].dtype != torch.float32), T, D, _dt(xs[0]), _stream())


# ----------------------------------------------------------------------------- pair rotation + page write
def rope_pairs_store(q: Tensor, k: Tensor, v: Tensor, inv_freq: Optional[Tensor], rot_dims: int, positions: Tensor,
                     seq_of: Tensor, block_table: Tensor, pool: Tensor, q_out: Tensor, n_heads: int,
                     n_kv_heads: int, dim: int, vdim: int, padded_dim: int, half_layout: bool = False,
                     biases: Optional[Tuple[Tensor, Tensor, Tensor]] = None,
                     qk_norm: Optional[Tuple[Tensor, Tensor, float]] = None) -> None:
    """Rotates pairs among the first ``rot_dims`` entries of every query and key head (neighbours
    (2i, 2i+1), or with ``half_layout`` entries (i, i + rot_dims/2)), writes queries to q_out [T, H*Dp]
    and keys and values into their pages [pages, 2, page, G*Dp], every head padded with zeros to Dp =
    ``padded_dim`` entries.  ``biases``: float vectors added to q, k and v as they are read.  ``qk_norm`` (weight
    [H*d], weight [G*d], eps): before rotation the token's whole query projection, and its whole key projection, is
    divided by its root mean square and multiplied by the weight (float); values are left as they are."""
    _cuda(q, k, v, inv_freq, positions, seq_of, block_table, pool, q_out)
    qn = kn = None
    norm_eps = 0.0
    if qk_norm is not None:
        qn, kn, norm_eps = qk_norm
        _cuda(qn, kn)
        _f32vec(qn, n_heads * dim, "rope_pairs_store: q norm weight")
        _f32vec(kn, n_kv_heads * dim, "rope_pairs_store: k norm weight")
    qb = kb = vb = None
    if biases is not None:
        qb, kb, vb = biases
        _f32vec(qb, n_heads * dim, "rope_pairs_store: q bias")
        _f32vec(kb, n_kv_heads * dim, "rope_pairs_store: k bias")
        _f32vec(vb, n_kv_heads * vdim, "rope_pairs_store: v bias")
    T = q.shape[0]
    ld_q, ld_k, ld_v = (_rows_view(t, "rope_pairs_store") for t in (q, k, v))
    if not (q.shape[1] == n_heads * dim and k.shape == (T, n_kv_heads * dim) and v.shape == (T, n_kv_heads * vdim)
            and q.dtype == k.dtype == v.dtype == pool.dtype == q_out.dtype):
        raise KernelError("rope_pairs_store: q [T, H*d], k [T, G*d], v [T, G*dv] of the pool's type")
    if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == n_kv_heads * padded_dim and pool.is_contiguous()
            and q_out.shape == (T, n_heads * padded_dim) and q_out.is_contiguous()):
        raise KernelError("rope_pairs_store: pool [pages, 2, page_size, G*Dp], q_out [T, H*Dp]")
    if rot_dims > 0:
        _f32vec(inv_freq, rot_dims // 2, "rope_pairs_store: inv_freq")
    _i32(positions, "rope_pairs_store: positions")
    _i32(seq_of, "rope_pairs_store: seq_of")
    _i32(block_table, "rope_pairs_store: block_table")
    _call("pmm_rope_pairs_store", q.data_ptr(), ld_q, k.data_ptr(), ld_k, v.data_ptr(), ld_v, _ptr(inv_freq),
          positions.data_ptr(), seq_of.data_ptr(), block_table.data_ptr(), block_table.shape[1], pool.data_ptr(),
          pool.shape[2], q_out.data_ptr(), T, n_heads, n_kv_heads, dim, vdim, padded_dim, int(rot_dims),
          int(bool(half_layout)), _ptr(qb), _ptr(kb), _ptr(vb), _ptr(qn), _ptr(kn), float(norm_eps), _dt(q), _stream())


# ----------------------------------------------------------------------------- matrix-state recurrences
RECURRENT_MAX_KEY_DIM = 256


def _recurrent_common(q: Tensor, k: Tensor, v: Tensor, state: Tensor, cu: Tensor, slots: Tensor, out: Tensor,
                      H: int, Hk: int, d: int, dv: int, what: str) -> Tuple[int, int, int, int]:
    T = q.shape[0]
    lds = tuple(_rows_view(t, what) for t in (q, k, v))
    if not (q.shape == (T, Hk * d) and k.shape == (T, Hk * d) and v.shape == (T, H * dv) and q.dtype == k.dtype == v.dtype):
        raise KernelError(f"{what}: q, k [T, Hk*d], v [T, H*dv] of one type")
    if not (state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, d, dv)):
        raise KernelError(f"{what}: state must be contiguous float32 [slots, H, d, dv]")
    if not (out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, H * dv)):
        raise KernelError(f"{what}: out must be contiguous float32 [T, H*dv]")
    if not (1 <= d <= RECURRENT_MAX_KEY_DIM):
        raise KernelError(f"{what}: key sizes up to {RECURRENT_MAX_KEY_DIM}")
    _i32(cu, f"{what}: cu_seqlens")
    _i32(slots, f"{what}: slots")
    return (T,) + lds


def delta_scan(q: Tensor, k: Tensor, v: Tensor, beta: Tensor, a: Tensor, dt_bias: Tensor, a_log: Tensor,
               state: Tensor, cu: Tensor, slots: Tensor, n_seq: int, out: Tensor, n_heads: int, n_qk_heads: int,
               dim: int, vdim: int, unit_eps: float, q_scale: float) -> None:
    """Gated delta rule, token by token, state [slots, H, d, dv] float32 carried between steps:
    S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q with g = exp(-exp(a_log_h)
    softplus(a + dt_bias)) per head and key channel, beta = sigmoid(beta_raw), q and k scaled to unit
    length (x / sqrt(sum x^2 + unit_eps); q also by q_scale)."""
    _cuda(q, k, v, beta, a, dt_bias, a_log, state, cu, slots, out)
    T, ld_q, ld_k, ld_v = _recurrent_common(q, k, v, state, cu, slots, out, n_heads, n_qk_heads, dim, vdim, "delta_scan")
    ld_b, ld_a = _rows_view(beta, "delta_scan: beta"), _rows_view(a, "delta_scan: a")
    if not (beta.shape == (T, n_heads) and a.shape == (T, n_heads * dim) and beta.dtype == a.dtype == q.dtype):
        raise KernelError("delta_scan: beta [T, H], a [T, H*d] of q's type")
    _f32vec(dt_bias, n_heads * dim, "delta_scan: dt_bias")
    _f32vec(a_log, n_heads, "delta_scan: a_log")
    _call("pmm_delta_scan", q.data_ptr(), ld_q, k.data_ptr(), ld_k, v.data_ptr(), ld_v, beta.data_ptr(), ld_b,
          a.data_ptr(), ld_a, dt_bias.data_ptr(), a_log.data_ptr(), state.data_ptr(), cu.data_ptr(), slots.data_ptr(),
          out.data_ptr(), int(n_seq), n_heads, n_qk_heads, dim, vdim, float(unit_eps), float(q_scale), _dt(q), _stream())


def decay_scan(q: Tensor, k: Tensor, v: Tensor, decay: Tensor, state: Tensor, cu: Tensor, slots: Tensor, n_seq: int,
               out: Tensor, n_heads: int, dim: int, vdim: int) -> None:
    """Linear attention with one decay per head, token by token: S <- decay_h S + k v^T; o = S^T q with
    q, k, v = silu of the given projections; state [slots, H, d, dv] float32 carried between steps."""
    _cuda(q, k, v, decay, state, cu, slots, out)
    T, ld_q, ld_k, ld_v = _recurrent_common(q, k, v, state, cu, slots, out, n_heads, n_heads, dim, vdim, "decay_scan")
    _f32vec(decay, n_heads, "decay_scan: decay")
    _call("pmm_decay_scan", q.data_ptr(), ld_q, k.data_ptr(), ld_k, v.data_ptr(), ld_v, decay.data_ptr(),
          state.data_ptr(), cu.data_ptr(), slots.data_ptr(), out.data_ptr(), int(n_seq), n_heads, dim, vdim, _dt(q),
          _stream())


RECURRENT_CHUNK = 64  # tokens per chunk of the chunked recurrences


def recurrent_chunked_supported(dim: int, delta: bool) -> bool:
    """Whether the chunked kernels take this key size (a multiple of 4 whose operands fit one block)."""
    return bool(_fn("pmm_recurrent_chunked_supported")(int(dim), int(bool(delta))))


def recurrent_chunks(new_lens: Sequence[int]) -> int:
    return sum((n + RECURRENT_CHUNK - 1) // RECURRENT_CHUNK for n in new_lens)


def recurrent_chunked_scratch_floats(new_lens: Sequence[int], n_heads: int, dim: int, vdim: int, delta: bool) -> int:
    f = _fn("pmm_recurrent_chunked_scratch")
    f.restype = c_longlong
    return recurrent_chunks(new_lens) * n_heads * int(f(int(dim), int(vdim), int(bool(delta)))) + 4


def recurrent_chunked(q: Tensor, k: Tensor, v: Tensor, state: Tensor, cu: Tensor, slots: Tensor, new_lens: Sequence[int],
                      out: Tensor, scratch: Tensor, n_heads: int, n_qk_heads: int, dim: int, vdim: int,
                      decay: Optional[Tensor] = None, beta: Optional[Tensor] = None, a: Optional[Tensor] = None,
                      dt_bias: Optional[Tensor] = None, a_log: Optional[Tensor] = None, unit_eps: float = 0.0,
                      q_scale: float = 1.0) -> None:
    """The recurrences of delta_scan (``decay`` None) and decay_scan (``decay`` given) for prompt portions,
    in chunks of 64 tokens: one launch prepares every chunk's operands in parallel, a second walks each
    sequence's chunks in order.  Float arithmetic throughout; same arguments and results (beyond rounding)
    as the token-serial kernels.  ``new_lens``: tokens per sequence (host values)."""
    delta = decay is None
    what = "recurrent_chunked"
    _cuda(q, k, v, decay, beta, a, dt_bias, a_log, state, cu, slots, out, scratch)
    T, ld_q, ld_k, ld_v = _recurrent_common(q, k, v, state, cu, slots, out, n_heads, n_qk_heads, dim, vdim, what)
    if not recurrent_chunked_supported(dim, delta):
        raise KernelError(f"{what}: key size {dim} is not one the chunked kernels take")
    ld_b = ld_a = 0
    if delta:
        ld_b, ld_a = _rows_view(beta, f"{what}: beta"), _rows_view(a, f"{what}: a")
        if not (beta.shape == (T, n_heads) and a.shape == (T, n_heads * dim) and beta.dtype == a.dtype == q.dtype):
            raise KernelError(f"{what}: beta [T, H], a [T, H*d] of q's type")
        _f32vec(dt_bias, n_heads * dim, f"{what}: dt_bias")
        _f32vec(a_log, n_heads, f"{what}: a_log")
    else:
        _f32vec(decay, n_heads, f"{what}: decay")
    need = recurrent_chunked_scratch_floats(new_lens, n_heads, dim, vdim, delta)
    if not (scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need):
        raise KernelError(f"{what}: needs {need} floats of scratch")
    base = scratch.data_ptr()
    base += (-base) % 16
    _call("pmm_recurrent_chunked", q.data_ptr(), ld_q, k.data_ptr(), ld_k, v.data_ptr(), ld_v, _ptr(beta), ld_b, _ptr(a),
          ld_a, _ptr(dt_bias), _ptr(a_log), _ptr(decay), state.data_ptr(), cu.data_ptr(), slots.data_ptr(), out.data_ptr(),
          base, len(new_lens), recurrent_chunks(new_lens), n_heads, n_qk_heads, dim, vdim, float(unit_eps), float(q_scale),
          _dt(q), _stream())


def ensure_built() -> str:
    """Build (if needed) and load the library; returns its path."""
    _build.load()
    return _build.library_path()
