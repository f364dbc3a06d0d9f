"""Python face of the CUDA kernel library (``csrc/``), loaded with ctypes.

Every function takes torch tensors that already live on the GPU, passes their addresses and the
current CUDA stream to an ``extern "C"`` launcher, and raises ``KernelError`` if the launcher
refuses the sizes or the launch fails. There is no CPU implementation behind these functions and
no library stand-in: if the shared library cannot be built or loaded, the first call raises.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

#: the gate functions that the products' gated epilogues know (act = f(gate) * up)
GATED_EPILOGUES = ("silu", "gelu_tanh")
#: how the unit epilogues are told to form gelu_tanh(gate) * up instead of the clamped unit: (limit, slope)
GELU_UNIT = (3.0e38, -1.0)

STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a cache slot or page id outside the pool",
               4: "a position outside the rotary table or beyond a block table", 8: "a bounded wait inside a kernel gave up"}


class KernelError(RuntimeError):
    pass


_lib = None
_lock = threading.Lock()
_c = ctypes
_P, _I, _LL, _F = _c.c_void_p, _c.c_int, _c.c_longlong, _c.c_float

_SIGNATURES = {
    "gb_embed": [_P, _I, _P, _P, _I, _I, _I, _F, _P, _P],
    "gb_rmsnorm": [_P, _P, _P, _P, _I, _I, _I, _F, _P],
    "gb_rope_kv_write": [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _LL, _I, _P, _P],
    "gb_swiglu": [_P, _P, _I, _I, _I, _P],
    "gb_copy_pages": [_P, _P, _P, _I, _LL, _LL, _LL, _LL, _I, _P],
    "gb_gemm_simt": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _LL, _LL, _LL, _P],
    "gb_attention_rows": [_P, _LL, _P, _LL, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_sample": [_P, _LL, _P, _P, _P, _P, _I, _P, _P, _I, _I, _P],
    "gb_resolve_tokens": [_P, _P, _P, _I, _I, _P],
    "gb_attention_decode": [_P, _LL, _P, _LL, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _I, _P, _P,
                            _P, _P, _P],
    "gb_attention_decode_counters": [_I, _I, _I],
    "gb_gemm_stream_row_groups": [_I, _I, _I, _I],
    "gb_gemm_stream": [_P, _LL, _P, _LL, _P, _F, _P, _LL, _P, _LL, _I, _I, _I, _I, _P, _LL, _I, _P],
    "gb_gemm_stream_qkv": [_P, _LL, _P, _LL, _P, _F, _P, _LL, _P, _LL, _I, _I, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I,
                           _LL, _I, _P, _P, _LL, _I, _P],
    "gb_attention_decode_mma_pdl": [_P, _LL, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _I, _P, _P,
                                    _P, _P, _I, _I, _I, _P],
    "gb_attention_decode_mma_sink": [_P, _LL, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _I, _P, _P,
                                     _P, _P, _I, _I, _I, _P, _P, _P, _P, _LL, _P],
    "gb_attention_decode_mma": [_P, _LL, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _I, _P, _P, _P,
                                _P, _P],
    "gb_attention_decode_mma_supported": [_I, _I, _I],
    "gb_stream_marker": [_P],
    "gb_kv_prefetch": [_P, _P, _P, _I, _P, _P, _I, _I, _I, _LL, _LL, _I, _I, _P],
    "gb_attention_prefill": [_P, _LL, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_attention_prefill_supported": [_I, _I, _I, _I],
    "gb_gemm_tcgen05_qkv": [_P, _P, _P, _I, _I, _LL, _LL, _LL, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _LL, _I, _P, _P,
                            _P, _I, _F],
    "gb_gemm_tcgen05_qkv_supported": [_I],
    "gb_attention_prefill_tc": [_P, _LL, _I, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_attention_prefill_tc_sink": [_P, _LL, _I, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P, _P,
                                     _P, _P, _LL, _P],
    "gb_attention_prefill_tc_supported": [_I, _I, _I, _I],
    "gb_gemm_tcgen05": [_P, _P, _P, _I, _I, _I, _I, _LL, _LL, _LL, _P, _P, _P, _P, _LL, _P, _P, _I, _F],
    "gb_gemm_tcgen05_column_tiles": [_I, _I, _I],
    "gb_gemm_tcgen05_supported": [_P, _P, _I, _I, _I, _LL, _LL],
    "gb_gemm_tcgen05_gated": [_P, _P, _P, _I, _I, _I, _LL, _LL, _LL, _P, _P, _P, _I, _F],
    "gb_gemm_tcgen05_unit": [_P, _P, _P, _I, _I, _I, _LL, _LL, _LL, _P, _P, _P, _F, _F],
    "gb_gemm_stream_unit": [_P, _LL, _P, _LL, _P, _F, _P, _LL, _P, _LL, _I, _I, _I, _P, _F, _F, _P, _LL, _I, _P],
    "gb_program_encode_gemm": [_P, _P, _LL, _P, _LL, _P, _F, _P, _LL, _P, _LL, _I, _I, _I, _I],
    "gb_program_encode_gemm_qkv": [_P, _P, _LL, _P, _LL, _P, _F, _P, _LL, _P, _LL, _I, _I, _P, _I, _P, _P, _P, _P, _I, _I, _I,
                                   _I, _LL, _I, _P],
    "gb_program_encode_attention": [_P, _P, _LL, _P, _LL, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _I, _P, _P,
                                    _P, _P, _I],
    "gb_program_launch": [_P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P],
    "gb_program_launch_with_absent_blocks": [_P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _LL, _P],
    "gb_program_launch_traced": [_P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _P],
    "gb_step_io": [_P, _P, _LL, _P, _P, _P, _LL, _P],
    "gb_rmsnorm_add": [_P, _LL, _P, _P, _LL, _I, _I, _F, _P, _P, _I, _P],
    "gb_cast_rows": [_P, _LL, _P, _P, _I, _I, _I, _P],
    "gb_add_bias": [_P, _LL, _P, _I, _I, _P],
    "gb_clamped_glu": [_P, _I, _LL, _P, _F, _F, _P, _I, _I, _I, _P],
    "gb_relu2": [_P, _P, _I, _LL, _P],
    "gb_scale": [_P, _LL, _F, _P],
    "gb_gated_head_norm": [_P, _P, _LL, _P, _P, _I, _I, _I, _I, _F, _I, _P],
    "gb_latent_kv_write": [_P, _LL, _I, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_latent_attention_rows": [_P, _P, _I, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_latent_attention_mma_supported": [_I, _I, _I],
    "gb_latent_attention_mma": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _I, _I,
                                _P, _P],
    "gb_head_linear_supported": [_P, _LL, _LL, _P, _P, _LL, _LL, _I, _I],
    "gb_head_linear": [_P, _LL, _LL, _P, _P, _LL, _LL, _I, _I, _I, _I, _P],
    "gb_embed_positions": [_P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P, _P],
    "gb_residual_conv": [_P, _I, _P, _I, _P, _P, _LL, _LL, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "gb_gelu_glu": [_P, _I, _LL, _P, _I, _I, _I, _P],
    "gb_scaled_sum": [_P, _P, _F, _F, _P, _LL, _I, _P],
    "gb_bias_rope_write": [_P, _LL, _P, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _LL, _I, _P, _P],
    "gb_talking_attention_rows": [_P, _P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _LL, _F, _F, _F, _I, _P, _P],
    "gb_talking_attention_decode": [_P, _P, _P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _LL, _F, _F, _F, _I, _I, _P, _P],
    "gb_talking_attention_decode_plan": [_I, _I, _I, _I],
    "gb_talking_attention_tiles": [_P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _LL, _F, _F, _F, _I, _P, _P],
    "gb_talking_attention_tiles_columns": [_I, _I, _I],
    "gb_talk_combine": [_P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _P],
    "gb_short_conv": [_P, _LL, _P, _P, _LL, _P, _LL, _LL, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "gb_channel_delta": [_P, _LL, _P, _LL, _P, _LL, _P, _P, _P, _LL, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _I, _P],
    "gb_channel_delta_decode_supported": [_I, _I],
    "gb_channel_delta_decode": [_P, _LL, _P, _LL, _P, _LL, _P, _P, _P, _LL, _P, _LL, _P, _F, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I,
                                _I, _I, _P, _P, _LL, _P, _LL, _I, _I, _I, _I, _P, _P, _I, _I, _I, _P],
    "gb_decay_linear_pieces": [_P, _LL, _P, _P, _LL, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _I, _I, _P, _P, _P],
    "gb_short_conv_state": [_P, _LL, _P, _LL, _LL, _P, _P, _P, _I, _I, _I, _I, _P],
    "gb_streams_broadcast": [_P, _P, _I, _I, _I, _P],
    "gb_streams_step": [_P, _I, _I, _P, _LL, _P, _P, _I, _P, _LL, _P, _P, _P, _P, _P, _P, _F, _P, _I, _P, _P, _P, _I, _I, _P],
    "gb_qk_norm_rope_write": [_P, _LL, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _LL, _I, _P, _P, _P, _LL,
                              _P, _P],
    "gb_sink_attention_rows": [_P, _P, _I, _P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _LL, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_sink_attention_decode": [_P, _P, _I, _P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _LL, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_sink_attention_decode_supported": [_I],
    "gb_sink_attention_tiles_supported": [_I, _I],
    "gb_sink_attention_tiles": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _LL, _I, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_sigmoid_attention_rows": [_P, _P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_sigmoid_attention_decode": [_P, _P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_sigmoid_attention_decode_supported": [_I],
    "gb_sigmoid_attention_tiles_supported": [_I, _I],
    "gb_sigmoid_attention_tiles": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _LL, _F, _I, _P, _P],
    "gb_mingru_scan": [_P, _LL, _P, _P, _P, _LL, _LL, _P, _LL, _I, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "gb_moe_route": [_P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P, _P, _P, _I, _P],
    "gb_moe_expert_rows": [_P, _I, _I, _P, _P, _I, _P, _P, _I, _I, _I, _P, _P],
    "gb_moe_expert_halves": [_P, _I, _I, _P, _P, _I, _P, _P, _I, _I, _I, _P, _P, _I, _F, _F, _P],
    "gb_moe_sort": [_P, _P, _I, _I, _I, _P, _P, _P, _P],
    "gb_moe_grouped_supported": [_I, _I],
    "gb_moe_grouped_gemm": [_P, _LL, _P, _I, _I, _P, _P, _P, _I, _I, _I, _P, _LL, _I, _I, _F, _F, _P],
    "gb_moe_combine": [_P, _P, _I, _P, _LL, _P, _P, _P, _LL, _I, _I, _I, _P],
    "gb_program_op_bytes": [],
    "gb_program_max_rows": [],
}


def lib():
    """The loaded shared library; builds it at first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.ensure_built()
            try:
                handle = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from None
            handle.gb_last_error.restype = ctypes.c_char_p
            handle.gb_last_error.argtypes = []
            for name, args in _SIGNATURES.items():
                fn = getattr(handle, name, None)
                if fn is None:
                    raise KernelError(f"{path} does not export {name}; rebuild it (csrc/build.py --force)")
                fn.argtypes = args
                fn.restype = ctypes.c_int
            handle.gb_set_pdl.argtypes = [ctypes.c_int]
            handle.gb_set_pdl.restype = None
            handle.gb_set_pdl(7 if USE_PDL else 0)
            _lib = handle
    return _lib


def step_io(host_meta_ptr: int, dev_meta: torch.Tensor, meta_bytes: int, graph_exec: int, sampled_dev: torch.Tensor,
            sampled_host: torch.Tensor, count: int, nodes: int) -> None:
    """A recorded decode step's traffic in one native call: metadata to the device, the graph, ``count`` sampled tokens
    back to pinned host memory; nothing is waited for. ``nodes``: the graph's kernel count, for ``launch_count``."""
    global launch_count
    rc = lib().gb_step_io(host_meta_ptr, dev_meta.data_ptr(), meta_bytes, graph_exec, sampled_dev.data_ptr(),
                          sampled_host.data_ptr(), 4 * count, _stream())
    if rc != 0:
        raise KernelError(lib().gb_last_error().decode("utf-8", "replace") or "gb_step_io failed")
    launch_count += nodes


def loaded_library_path() -> Optional[str]:
    return _build.library_path() if _lib is not None else None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


#: kernels launched through this module since import (graph replays add their node count)
launch_count = 0


def _call(name: str, *args) -> None:
    global launch_count
    if _program is not None:
        _program.flush()          # a kernel that is launched now must come after what was recorded before it
    launch_count += 1
    rc = getattr(lib(), name)(*args)
    if rc != 0:
        raise KernelError(lib().gb_last_error().decode("utf-8", "replace") or f"{name} failed with code {rc}")


# -------------------------------------------------------------------------------------- decode programs
BY_ROWS, BY_OPERATIONS = 0, 1
#: the default way in which a program's persistent kernel shares the work (see ``Program.how``)
PROGRAM_HOW = BY_ROWS


class Program:
    """A chain of small decode kernels written down as operations and run by one persistent kernel
    (``csrc/decode_program.cu``). While a program is open (``program_begin`` .. ``program_end``), the products of at
    most ``max_rows`` rows that ``gemm_stream`` / ``gemm_stream_qkv`` would launch and the attention that
    ``attention_decode_mma`` would launch are appended to it instead; any other kernel launched through this module
    first runs what has been recorded so far, so the order of the work never changes. Nothing here knows what the
    operations belong to: parts call the same functions as ever.

    A program object remembers the operation arrays it has run (one per flush of a step, in order). When a step
    records exactly the same operations again (same buffers, same shapes: the second run of a step that is being
    recorded into a CUDA graph, or the next step of the same shape), the copy on the device is reused."""

    def __init__(self):
        handle = lib()
        self.op_bytes = int(handle.gb_program_op_bytes())
        self.max_rows = int(handle.gb_program_max_rows())
        self.segments = []
        self.cursor = 0
        self.absent_blocks, self.wait_cycles = 0, 0
        self.trace_next, self.traces = False, []
        #: how the persistent kernel shares the work: BY_ROWS (a thread-block cluster per group of rows runs the whole
        #: program for them) or BY_OPERATIONS (all resident blocks share each operation and meet at a barrier)
        self.how = PROGRAM_HOW
        self._buf = ctypes.create_string_buffer(self.op_bytes)
        self._reset()

    def _reset(self):
        self._pending, self._n, self._rows, self._hd, self._bk, self._max_vblocks, self._max_k = [], 0, 0, 0, 0, 1, 8
        self._status = None

    def start_step(self):
        self.cursor = 0
        self._reset()

    def _add(self, name, vblocks, rows, k, *args):
        rc = getattr(lib(), name)(ctypes.addressof(self._buf), *args)
        if rc != 0:
            raise KernelError(lib().gb_last_error().decode("utf-8", "replace") or f"{name} failed with code {rc}")
        self._pending.append(self._buf.raw)
        self._n += 1
        self._rows = max(self._rows, rows)
        self._max_vblocks = max(self._max_vblocks, vblocks)
        self._max_k = max(self._max_k, k)

    #: a product whose weights are larger than this is launched by itself (all SMs stream it) instead of recorded: in a
    #: program shared by rows a cluster would have to stream it alone
    MAX_WEIGHT_BYTES = 12 << 20

    def takes_rows(self, rows: int) -> bool:
        return 1 <= rows <= self.max_rows

    def takes_product(self, rows: int, w: torch.Tensor) -> bool:
        return self.takes_rows(rows) and w.numel() * w.element_size() <= self.MAX_WEIGHT_BYTES

    def takes_attention(self, hd: int, block_keys: int) -> bool:
        """One program runs one attention variant; a second one waits for the next program."""
        bk = 16 if (hd == 64 and block_keys == 16) or hd == 128 else 32
        return self._hd in (0, hd) and (self._hd == 0 or self._bk == bk)

    def flush(self) -> None:
        """Run what has been recorded (one launch) and start an empty recording."""
        global launch_count
        if not self._n:
            return
        host = b"".join(self._pending)
        n, rows, hd, bk, max_vblocks, max_k, status = (self._n, self._rows, self._hd, self._bk, self._max_vblocks, self._max_k,
                                                        self._status)
        self._reset()
        k = self.cursor
        if k < len(self.segments) and self.segments[k]["host"] == host:
            seg = self.segments[k]
        else:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("a decode program changed between the run that prepared a CUDA graph and its recording")
            dev = torch.empty(len(host), dtype=torch.uint8, device=status.device)
            dev.copy_(torch.frombuffer(bytearray(host), dtype=torch.uint8))
            seg = {"host": host, "dev": dev, "barrier": torch.zeros(1, dtype=torch.int32, device=status.device)}
            del self.segments[k:]
            self.segments.append(seg)
        self.cursor = k + 1
        launch_count += 1
        if self.trace_next:        # (a measurement: per-operation clock values of the first and the last block)
            self.traces.append((n, torch.zeros(2 * n * 4, dtype=torch.int64, device=status.device), host))
            rc = lib().gb_program_launch_traced(seg["dev"].data_ptr(), n, rows, hd, bk, max_vblocks, max_k, seg["barrier"].data_ptr(),
                                                status.data_ptr(), self.how, self.traces[-1][1].data_ptr(), _stream())
        elif self.absent_blocks:     # (a test of the barrier's bounded wait)
            rc = lib().gb_program_launch_with_absent_blocks(seg["dev"].data_ptr(), n, rows, hd, bk, max_vblocks, max_k,
                                                            seg["barrier"].data_ptr(), status.data_ptr(), self.absent_blocks,
                                                            self.wait_cycles, _stream())
        else:
            rc = lib().gb_program_launch(seg["dev"].data_ptr(), n, rows, hd, bk, max_vblocks, max_k, seg["barrier"].data_ptr(),
                                         status.data_ptr(), self.how, _stream())
        if rc != 0:
            raise KernelError(lib().gb_last_error().decode("utf-8", "replace") or f"gb_program_launch failed with code {rc}")


_program: Optional[Program] = None


def program_begin(program: Program, status: torch.Tensor) -> None:
    """Start recording into ``program``; ``status`` is the device status word its kernel reports to."""
    global _program
    if _program is not None:
        raise KernelError("a decode program is already being recorded")
    program.start_step()
    program._status = status
    program._default_status = status
    _program = program


def program_end() -> None:
    """Run what is still recorded and stop recording."""
    global _program
    if _program is not None:
        try:
            _program.flush()
        finally:
            _program = None


def _program_for(status: Optional[torch.Tensor] = None) -> Optional[Program]:
    p = _program
    if p is not None and p._status is None:
        p._status = status if status is not None else p._default_status
    return p


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported tensor dtype {t.dtype}") from None


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operands must be CUDA tensors; there is no CPU path")


def check_status(status: torch.Tensor) -> None:
    """Read the device status word (synchronises) and raise if a kernel recorded a bad index."""
    bits = int(status.item())
    if bits:
        status.zero_()
        what = [msg for bit, msg in STATUS_BITS.items() if bits & bit]
        raise KernelError("a kernel skipped an access: " + "; ".join(what))


# ------------------------------------------------------------------------------------------ ops
def embed(table: torch.Tensor, tokens: torch.Tensor, x: torch.Tensor, status: torch.Tensor, scale: float = 1.0) -> None:
    """x[i, :] = table[tokens[i], :] * scale as float32."""
    _cuda(table, tokens, x, status)
    n, d = x.shape
    assert tokens.dtype == torch.int32 and x.dtype == torch.float32 and x.is_contiguous() and table.is_contiguous()
    _call("gb_embed", _ptr(table), _dt(table), _ptr(tokens), _ptr(x), n, d, table.shape[0], float(scale), _ptr(status), _stream())


def embed_positions(table: torch.Tensor, pos_table: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor, x: torch.Tensor,
                    status: torch.Tensor) -> None:
    """x[i, :] = table[tokens[i], :] + pos_table[positions[i], :], summed in float32; padding rows (position < 0) are cleared."""
    _cuda(table, pos_table, tokens, positions, x, status)
    n, d = x.shape
    assert table.dtype == pos_table.dtype and table.shape[1] == pos_table.shape[1] == d and x.dtype == torch.float32
    assert table.is_contiguous() and pos_table.is_contiguous() and x.is_contiguous() and tokens.shape[0] >= n and positions.shape[0] >= n
    _call("gb_embed_positions", _ptr(table), _ptr(pos_table), _dt(table), _ptr(tokens), _ptr(positions), _ptr(x), n, d, table.shape[0],
          pos_table.shape[0], _ptr(status), _stream())


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = gain * x[rows[r] or r, :] / sqrt(mean(x^2) + eps); x and gain float32."""
    _cuda(x, gain, out, rows)
    assert x.dtype == torch.float32 and gain.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    n, d = out.shape
    assert x.shape[1] == d and gain.numel() == d
    _call("gb_rmsnorm", _ptr(x), _ptr(rows), _ptr(gain), _ptr(out), _dt(out), n, d, float(eps), _stream())


def rope_kv_write(qkv: torch.Tensor, cos_sin: Optional[torch.Tensor], positions: torch.Tensor, slots: torch.Tensor,
                  kcache: torch.Tensor, vcache: torch.Tensor, nh: int, nkv: int, hd: int, rot: int,
                  page_size: int, write_kv: bool, status: torch.Tensor) -> None:
    """Rotate q and k of each row at its position (in place) and store k, v at the row's slot.
    kcache/vcache: [pages, nkv, page_size, hd]; cos_sin: float32 [max_pos, rot/2, 2]."""
    _cuda(qkv, cos_sin, positions, slots, kcache, vcache, status)
    n = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * hd
    assert kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype and kcache.is_contiguous() and vcache.is_contiguous()
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    _call("gb_rope_kv_write", _ptr(qkv), _dt(qkv), _ptr(cos_sin), _ptr(positions), _ptr(slots), _ptr(kcache),
          _ptr(vcache), n, nh, nkv, hd, rot if cos_sin is not None else 0, max_pos, page_size, kcache.shape[0],
          1 if write_kv else 0, _ptr(status), _stream())


def swiglu(gate_up: torch.Tensor, act: torch.Tensor) -> None:
    _cuda(gate_up, act)
    n, inter = act.shape
    assert gate_up.shape == (n, 2 * inter) and gate_up.dtype == act.dtype
    assert gate_up.is_contiguous() and act.is_contiguous()
    _call("gb_swiglu", _ptr(gate_up), _ptr(act), _dt(act), n, inter, _stream())


def copy_pages(kcache: torch.Tensor, vcache: torch.Tensor, pairs: torch.Tensor) -> None:
    """kcache/vcache: [layers, pages, ...]; pairs int32 [n, 2] of (source page, destination page)."""
    _cuda(kcache, vcache, pairs)
    layers = kcache.shape[0]
    layer_bytes = kcache.stride(0) * kcache.element_size()
    page_bytes = kcache.stride(1) * kcache.element_size()
    has_v = vcache.numel() > 0       # (a group that keeps one tensor per token has an empty second pool)
    _call("gb_copy_pages", _ptr(kcache), _ptr(vcache) if has_v else 0, _ptr(pairs), pairs.shape[0], page_bytes, layer_bytes,
          vcache.stride(1) * vcache.element_size() if has_v else 0, vcache.stride(0) * vcache.element_size() if has_v else 0,
          layers, _stream())


def gemm_simt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, accumulate: bool = False) -> None:
    """c[M, N] (+)= a[M, K] @ w[N, K]^T with float32 FMA on the CUDA cores (rows may be strided)."""
    _cuda(a, w, c)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    _call("gb_gemm_simt", _ptr(a), _dt(a), _ptr(w), _dt(w), _ptr(c), _dt(c), 1 if accumulate else 0, M, N, K,
          a.stride(0), w.stride(0), c.stride(0), _stream())


STREAM_MAX_ROWS = 64
#: above this many rows the norm is not folded into the stream kernels (every block would repeat
#: the normalisation of all rows) and QKV keeps one strip per block (twice the blocks) -- unless the
#: kernel takes the rows in groups of eight (``stream_folds``)
STREAM_FUSE_MAX_ROWS = 16


def stream_row_groups(rows: int, w: torch.Tensor) -> int:
    """In how many groups of eight rows the weight-streaming kernel runs a product of ``rows`` rows with ``w`` (1: all
    rows in one group). Small matrices are taken group by group: every block then works as for eight rows."""
    return int(lib().gb_gemm_stream_row_groups(rows, w.shape[0], w.shape[1], 0))


def stream_folds(rows: int, w: torch.Tensor) -> bool:
    """Whether a norm in front of this product (and rotation and the cache write behind a QKV product) is folded into
    the weight-streaming kernel: with few rows, or when the rows go in groups of eight."""
    return rows <= STREAM_FUSE_MAX_ROWS or (rows <= STREAM_MAX_ROWS and stream_row_groups(rows, w) > 1)


#: launch the decode-path kernels under programmatic stream serialisation (they wait for their
#: predecessor themselves, after work that does not depend on it)
USE_PDL = True


def gemm_stream_supported(a, w: torch.Tensor, rows: Optional[int] = None) -> bool:
    """Whether the weight-streaming kernel (few rows, bfloat16 weights) takes these operands. ``a``
    is a bfloat16 [M, K] tensor, or a float32 one that the kernel normalises on the way in."""
    M, K = a.shape
    if w.dtype != torch.bfloat16 or M > STREAM_MAX_ROWS or K % 8 or w.stride(0) % 8 or w.data_ptr() % 16:
        return False
    if a.dtype == torch.bfloat16:
        return a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
    return a.dtype == torch.float32 and a.stride(0) % 4 == 0 and a.data_ptr() % 16 == 0


def _stream_input(a: torch.Tensor, norm):
    """(x, ldx, xres, ldr, gain, eps) for the stream kernels: bfloat16 activations as they are, or
    float32 rows with the (gain, eps) of an RMSNorm to apply on the way in."""
    if norm is None:
        assert a.dtype == torch.bfloat16
        return _ptr(a), a.stride(0), 0, 0, 0, 0.0
    gain, eps = norm
    assert a.dtype == torch.float32 and gain.dtype == torch.float32 and gain.numel() == a.shape[1]
    return 0, 0, _ptr(a), a.stride(0), _ptr(gain), float(eps)


def _prefetch_args(t: Optional[torch.Tensor]):
    return (0, 0) if t is None else (t.data_ptr(), t.numel() * t.element_size())


def gemm_stream(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, accumulate: bool = False, gated: bool = False,
                norm=None, prefetch: Optional[torch.Tensor] = None, relu2: bool = False) -> None:
    """c[M, N] (+)= a[M, K] @ w[N, K]^T for M <= 64 on the tensor cores, streaming w once. With
    ``gated``, w is [2I, K] (gate rows, then up rows) and c[M, I] = silu(a gate^T) * (a up^T). With
    ``norm`` = (gain, eps), ``a`` is the float32 residual and is RMS-normalised on the way in.
    ``prefetch`` names a tensor (a later kernel's weights) to pull into L2 meanwhile."""
    _cuda(a, w, c)
    M, K = a.shape
    N = w.shape[0] // 2 if gated else w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    if gated:
        assert c.dtype == torch.bfloat16 and not accumulate
        mode = 3
    elif relu2:                      # c = bfloat16(max(a w^T, 0)^2)
        assert c.dtype == torch.bfloat16 and not accumulate
        mode = 5
    elif accumulate:
        assert c.dtype == torch.float32
        mode = 2
    else:
        mode = 0 if c.dtype == torch.bfloat16 else 1
        assert c.dtype in (torch.bfloat16, torch.float32)
    x, ldx, xres, ldr, gain, eps = _stream_input(a, norm)
    prog = _program_for()
    if prog is not None and prog.takes_product(M, w):
        prog._add("gb_program_encode_gemm", -(-N // 16), M, K, x, ldx, xres, ldr, gain, eps, _ptr(w), w.stride(0), _ptr(c),
                  c.stride(0), mode, M, N, K)
        return
    _call("gb_gemm_stream", x, ldx, xres, ldr, gain, eps, _ptr(w), w.stride(0), _ptr(c), c.stride(0), mode, M, N, K,
          *_prefetch_args(prefetch), 1 if USE_PDL else 0, _stream())


def gemm_stream_qkv_supported(a, w: torch.Tensor, hd: int, q_out: torch.Tensor) -> bool:
    return (gemm_stream_supported(a, w) and stream_folds(a.shape[0], w) and hd % 32 == 0
            and q_out.dtype == torch.bfloat16)


def gemm_stream_qkv(a: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cos_sin: Optional[torch.Tensor],
                    positions: torch.Tensor, slots: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, nh: int,
                    nkv: int, hd: int, page_size: int, write_kv: bool, status: torch.Tensor, norm=None,
                    prefetch: Optional[torch.Tensor] = None) -> None:
    """Stacked QKV projection for M <= 64 with rotary encoding and the cache write in its epilogue:
    q_out[:, :nh*hd] receives the rotated queries, rotated keys and values go to each row's cache slot.
    Full rotary (table [max_pos, hd/2, 2]) or none (cos_sin None)."""
    _cuda(a, w, q_out, cos_sin, positions, slots, kcache, vcache, status)
    M, K = a.shape
    assert w.shape == ((nh + 2 * nkv) * hd, K) and q_out.stride(1) == 1 and q_out.shape[0] == M
    assert kcache.dtype == vcache.dtype == torch.bfloat16 and kcache.is_contiguous() and vcache.is_contiguous()
    if cos_sin is not None:
        assert cos_sin.shape[1] == hd // 2
    x, ldx, xres, ldr, gain, eps = _stream_input(a, norm)
    prog = _program_for(status)
    if prog is not None and prog.takes_product(M, w):
        prog._add("gb_program_encode_gemm_qkv", (nh + 2 * nkv) * (hd // 32), M, K, x, ldx, xres, ldr, gain, eps, _ptr(w),
                  w.stride(0), _ptr(q_out), q_out.stride(0), M, K, _ptr(cos_sin),
                  cos_sin.shape[0] if cos_sin is not None else 0, _ptr(positions), _ptr(slots), _ptr(kcache), _ptr(vcache),
                  nh, nkv, hd, page_size, kcache.shape[0], 1 if write_kv else 0, _ptr(status))
        return
    _call("gb_gemm_stream_qkv", x, ldx, xres, ldr, gain, eps, _ptr(w), w.stride(0), _ptr(q_out), q_out.stride(0), M, K,
          _ptr(cos_sin), cos_sin.shape[0] if cos_sin is not None else 0, _ptr(positions), _ptr(slots), _ptr(kcache),
          _ptr(vcache), nh, nkv, hd, page_size, kcache.shape[0], 1 if write_kv else 0, _ptr(status),
          *_prefetch_args(prefetch), 1 if USE_PDL else 0, _stream())


def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes these operands (bfloat16, TMA-aligned)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or c.dtype not in (torch.bfloat16, torch.float32):
        return False
    return bool(lib().gb_gemm_tcgen05_supported(_ptr(a), _ptr(w), a.shape[0], w.shape[0], a.shape[1], a.stride(0),
                                                w.stride(0)))


_tc_status = {}


class RowScale:
    """The consumer half of an RMSNorm split between two tile-kernel products: ``ss`` float32 [M, parts] holds partial
    sums of squares of the residual rows, and each row of the product is multiplied by
    1 / sqrt(sum(ss[row]) / K + eps). The product's ``a`` operand is then bfloat16(residual * gain)."""
    __slots__ = ("ss", "eps")

    def __init__(self, ss: torch.Tensor, eps: float):
        assert ss.dtype == torch.float32 and ss.dim() == 2 and ss.is_contiguous()
        self.ss, self.eps = ss, float(eps)

    def args(self, rows: int):
        assert self.ss.shape[0] == rows
        return _ptr(self.ss), self.ss.shape[1], self.eps


_NO_SCALE = (None, 0, 0.0)


def gemm_tc_column_tiles(rows: int, n: int, k: int) -> int:
    """Column tiles of the output of a ``gemm_tc`` that adds [rows, k] x [n, k]^T into float32: the second extent of
    the partial sums of squares that a product with ``prepare`` writes."""
    return int(lib().gb_gemm_tcgen05_column_tiles(rows, n, k))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, accumulate: bool = False,
            status: Optional[torch.Tensor] = None, prepare=None, row_scale: Optional[RowScale] = None, relu2: bool = False) -> None:
    """c[M, N] (+)= a[M, K] @ w[N, K]^T with TMA + tcgen05.mma + TMEM. ``status`` receives the
    wait-timeout bit if a bounded wait inside the kernel ever gives up.

    ``prepare=(gain, pre, ss)`` (only with ``accumulate``) makes the epilogue the producer half of an RMSNorm of the
    rows it has just completed: ``pre`` bfloat16 [M, N] receives c * gain and ``ss`` float32
    [M, gemm_tc_column_tiles(M, N, K)] the partial sums of squares; a later product takes ``pre`` as its ``a`` with
    ``row_scale=RowScale(ss, eps)``."""
    _cuda(a, w, c, status)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    prep = (None, None, 0, None)
    if prepare is not None:
        gain, pre, ss = prepare
        _cuda(gain, pre, ss)
        assert accumulate and gain.dtype == torch.float32 and gain.numel() == N and gain.is_contiguous()
        assert pre.dtype == torch.bfloat16 and pre.shape == (M, N) and pre.stride(1) == 1
        assert ss.dtype == torch.float32 and ss.is_contiguous() and ss.shape == (M, gemm_tc_column_tiles(M, N, K))
        prep = (_ptr(gain), _ptr(pre), pre.stride(0), _ptr(ss))
    if status is None:
        status = _tc_status.get(a.device)
        if status is None:
            status = _tc_status[a.device] = torch.zeros(1, dtype=torch.int32, device=a.device)
    if relu2:                        # c = bfloat16(max(a w^T, 0)^2)
        assert c.dtype == torch.bfloat16 and not accumulate
        mode = 4
    elif accumulate:
        assert c.dtype == torch.float32
        mode = 2
    else:
        mode = 0 if c.dtype == torch.bfloat16 else 1
    _call("gb_gemm_tcgen05", _ptr(a), _ptr(w), _ptr(c), mode, M, N, K, a.stride(0), w.stride(0), c.stride(0),
          _ptr(status), _stream(), *prep, *(row_scale.args(M) if row_scale is not None else _NO_SCALE))


def gemm_tc_qkv_supported(a: torch.Tensor, w: torch.Tensor, hd: int, q_out: torch.Tensor, kcache: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel can project, rotate and write the cache in one go for these operands."""
    return (q_out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and q_out.stride(0) % 8 == 0
            and q_out.data_ptr() % 16 == 0 and bool(lib().gb_gemm_tcgen05_qkv_supported(hd)) and gemm_tc_supported(a, w, q_out))


def gemm_tc_qkv(a: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cos_sin: Optional[torch.Tensor],
                positions: torch.Tensor, slots: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, nh: int, nkv: int,
                hd: int, page_size: int, write_kv: bool, status: torch.Tensor, row_scale: Optional[RowScale] = None) -> None:
    """Stacked QKV projection on the tcgen05 kernel with the rotation and the cache write in its epilogue:
    q_out[:, :nh*hd] receives the rotated queries, the cache slots of the rows the rotated keys and the
    values. ``cos_sin`` is float32 [max_pos, hd/2, 2] or None (no rotation). ``row_scale``: see ``RowScale``."""
    _cuda(a, w, q_out, cos_sin, positions, slots, kcache, vcache, status)
    M, K = a.shape
    assert w.shape == ((nh + 2 * nkv) * hd, K) and a.stride(1) == 1 and w.stride(1) == 1 and q_out.stride(1) == 1
    assert q_out.shape[0] == M and q_out.shape[1] >= nh * hd and kcache.is_contiguous() and vcache.is_contiguous()
    assert cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape[1:] == (hd // 2, 2) and cos_sin.is_contiguous())
    _call("gb_gemm_tcgen05_qkv", _ptr(a), _ptr(w), _ptr(q_out), M, K, a.stride(0), w.stride(0), q_out.stride(0),
          _ptr(cos_sin), cos_sin.shape[0] if cos_sin is not None else 0, _ptr(positions), _ptr(slots), _ptr(kcache),
          _ptr(vcache), nh, nkv, hd, page_size, kcache.shape[0], 1 if write_kv else 0, _ptr(status), _stream(),
          *(row_scale.args(M) if row_scale is not None else _NO_SCALE))


def gemm_tc_gated(a: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor,
                  status: Optional[torch.Tensor] = None, row_scale: Optional[RowScale] = None) -> None:
    """act[M, I] = silu(a gate^T) * (a up^T) with w_gate_up = [gate rows; up rows], on the tcgen05
    kernel: gate and up columns of a tile sit side by side in one TMEM accumulator. ``row_scale``: see ``RowScale``."""
    _cuda(a, w_gate_up, act, status)
    M, K = a.shape
    inter = w_gate_up.shape[0] // 2
    assert w_gate_up.shape == (2 * inter, K) and act.shape == (M, inter) and act.dtype == torch.bfloat16
    assert a.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1
    if status is None:
        status = _tc_status.get(a.device)
        if status is None:
            status = _tc_status[a.device] = torch.zeros(1, dtype=torch.int32, device=a.device)
    _call("gb_gemm_tcgen05_gated", _ptr(a), _ptr(w_gate_up), _ptr(act), M, inter, K, a.stride(0), w_gate_up.stride(0),
          act.stride(0), _ptr(status), _stream(), *(row_scale.args(M) if row_scale is not None else _NO_SCALE))


def gemm_tc_unit(a: torch.Tensor, w_gate_up: torch.Tensor, bias: Optional[torch.Tensor], limit: float, slope: float,
                 act: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """``gemm_tc_gated`` with the clamped unit in the epilogue: act[M, I] = g * sigmoid(slope * g) * (u + 1) with
    g = min(a gate^T + bias[:I], limit) and u = clamp(a up^T + bias[I:], -limit, limit), from the float32 sums in TMEM.
    ``bias`` float32 [2 I] or None."""
    _cuda(a, w_gate_up, act, bias, status)
    M, K = a.shape
    inter = w_gate_up.shape[0] // 2
    assert w_gate_up.shape == (2 * inter, K) and act.shape == (M, inter) and act.dtype == torch.bfloat16
    assert a.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == 2 * inter and bias.is_contiguous())
    if status is None:
        status = _tc_status.get(a.device)
        if status is None:
            status = _tc_status[a.device] = torch.zeros(1, dtype=torch.int32, device=a.device)
    _call("gb_gemm_tcgen05_unit", _ptr(a), _ptr(w_gate_up), _ptr(act), M, inter, K, a.stride(0), w_gate_up.stride(0),
          act.stride(0), _ptr(status), _stream(), _ptr(bias), float(limit), float(slope))


def gemm_stream_unit(a: torch.Tensor, w_gate_up: torch.Tensor, bias: Optional[torch.Tensor], limit: float, slope: float,
                     act: torch.Tensor, prefetch: Optional[torch.Tensor] = None) -> None:
    """The gated form of ``gemm_stream`` (at most 64 rows, the weights streamed once) with the clamped unit of
    ``gemm_tc_unit`` in its epilogue; the number of units must be a multiple of 16."""
    _cuda(a, w_gate_up, act, bias)
    M, K = a.shape
    inter = w_gate_up.shape[0] // 2
    assert w_gate_up.shape == (2 * inter, K) and act.shape == (M, inter) and act.dtype == torch.bfloat16
    assert a.dtype == torch.bfloat16 and a.stride(1) == 1 and w_gate_up.stride(1) == 1 and act.stride(1) == 1
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == 2 * inter and bias.is_contiguous())
    x, ldx, xres, ldr, gain, eps = _stream_input(a, None)
    _call("gb_gemm_stream_unit", x, ldx, xres, ldr, gain, eps, _ptr(w_gate_up), w_gate_up.stride(0), _ptr(act), act.stride(0),
          M, inter, K, _ptr(bias), float(limit), float(slope), *_prefetch_args(prefetch), 1 if USE_PDL else 0, _stream())


def attention_rows(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                   block_tables: torch.Tensor, row_seq: torch.Tensor, positions: torch.Tensor, nh: int, nkv: int,
                   hd: int, page_size: int, scale: float, window: Optional[int], status: torch.Tensor) -> None:
    """One warp per (row, head): softmax(q k^T * scale) v over the row's visible keys."""
    _cuda(q, out, kcache, vcache, block_tables, row_seq, positions, status)
    n = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == kcache.dtype
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    _call("gb_attention_rows", _ptr(q), q.stride(0), _ptr(out), out.stride(0), _dt(q), _ptr(kcache), _ptr(vcache),
          _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), _ptr(positions), n, nh, nkv, hd, page_size,
          kcache.shape[0], float(scale), int(window or 0), _ptr(status), _stream())


DECODE_KEYS_PER_TILE = 64


def decode_splits(n: int, nh: int, nkv: int, max_context: int, target_blocks: int = 148 * 4) -> int:
    """How many blocks share the keys of one (row, kv head): enough to fill the GPU, never more than
    there are 64-key tiles. Depends on the batch shape only, so a captured graph can fix it."""
    per_split = lib().gb_attention_decode_counters(n, nh, nkv)
    tiles = max(1, -(-max_context // DECODE_KEYS_PER_TILE))
    return max(1, min(-(-target_blocks // max(per_split, 1)), tiles))


def attention_decode(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                     block_tables: torch.Tensor, row_seq: torch.Tensor, positions: torch.Tensor, nh: int, nkv: int,
                     hd: int, page_size: int, scale: float, window: Optional[int], splits: int,
                     part_acc: Optional[torch.Tensor], part_ml: Optional[torch.Tensor],
                     counters: Optional[torch.Tensor], status: torch.Tensor) -> None:
    """Split-key attention for rows with few queries per request. Scratch (needed when splits > 1):
    part_acc float32 [n, nh, splits, hd], part_ml float32 [n, nh, splits, 2], counters int32
    [gb_attention_decode_counters(n, nh, nkv)] that are zero on entry and left zero."""
    _cuda(q, out, kcache, vcache, block_tables, row_seq, positions, part_acc, part_ml, counters, status)
    n = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == kcache.dtype
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    if splits > 1:
        assert part_acc.numel() >= n * nh * splits * hd and part_ml.numel() >= n * nh * splits * 2
        assert counters.numel() >= lib().gb_attention_decode_counters(n, nh, nkv)
    _call("gb_attention_decode", _ptr(q), q.stride(0), _ptr(out), out.stride(0), _dt(q), _ptr(kcache), _ptr(vcache),
          _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), _ptr(positions), n, nh, nkv, hd, page_size,
          kcache.shape[0], float(scale), int(window or 0), int(splits), _ptr(part_acc), _ptr(part_ml),
          _ptr(counters), _ptr(status), _stream())


def attention_decode_mma_supported(dtype: torch.dtype, nh: int, nkv: int, hd: int, page_size: int = 16) -> bool:
    return (dtype == torch.bfloat16 and page_size >= 16 and page_size & (page_size - 1) == 0
            and bool(lib().gb_attention_decode_mma_supported(nh, nkv, hd)))


DECODE_MMA_WAVE_SINGLE = 444        # blocks of the 16-key, four-warp variant that run at once: 148 SMs x 3
DECODE_MMA_WAVE_BLOCKS = 410        # the same in clusters of 2 to 4 (measured: 410 fit, 432 do not)
DECODE_MMA_BLOCK_US = 5.7           # a block's fixed cost, microseconds (measured)
DECODE_MMA_KEY_US = 0.0147          # and its cost per key


def decode_mma_plan(n: int, nkv: int, hd: int, max_context: int):
    """(splits, keys per warp iteration, warps per block) for the tensor-core decode kernel. A small batch needs
    many blocks per (row, kv head) to fill the GPU, but each block keeps at least 512 keys, below which the
    fixed cost of a block and of the merge outweighs the parallelism; where that leaves at most one block
    per SM, a block has eight warps instead of four, so that each warp walks through half as many keys (the
    splits are then rounded down: a second block of eight warps does not fit beside the first). A batch that
    fills the GPU by itself takes the 16-key variant (three blocks per SM instead of two) and the split count
    whose waves of resident blocks are estimated to end soonest.
    Depends on the batch shape and the longest context the step allows, never on the data, so a captured
    graph can fix it."""
    pairs = max(n * nkv, 1)
    most = max(1, -(-max_context // 512))
    if hd == 64 and pairs >= 96:
        # Blocks of the 16-key variant run three to an SM, in waves: all blocks of a wave take as long as one of them.
        # A block costs about 5.7 us of start, merge and hand-over and 14.7 ns a key; a wave holds about 410 blocks
        # (432 no longer fit one; without clusters, at one split, 416 still do: 71.3 us, 3 splits 92.0). The split count that this estimate likes best, among 1 to 4 (clusters of 5 and 7
        # place badly), is the one measured best at context 4096 for 96 to 2,048 pairs, within 1 %: 128 pairs 3 splits
        # 26.8 us (2: 34.6, 4: 37.3); 144 pairs 2 splits 35.6 (3: 45.6); 256 pairs 3 splits 51.6 (1: 66.1, 2: 66.3,
        # 4: 57.7); 320 pairs 1 split 68.4 (2: 72.9, 4: 79.0); 512 pairs 3 splits 99.0 (1: 123.1, 4: 98.2); 2,048 pairs
        # 1 split 338.7 (2: 354.7). (Filling two blocks per SM once, the rule before, took 2 splits at 256 pairs: a 1.7B
        # decode step at batch 8 2.85 ms, with 3 splits 2.56 ms.)
        best, best_cost = 1, None
        for splits in range(1, min(4, most) + 1):
            waves = -(-pairs * splits // (DECODE_MMA_WAVE_BLOCKS if splits > 1 else DECODE_MMA_WAVE_SINGLE))
            cost = waves * (DECODE_MMA_BLOCK_US + DECODE_MMA_KEY_US * -(-max_context // splits))
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = splits, cost
        return best, 16, 4
    if hd == 64 and pairs <= 74:
        # (measured at 9/3 heads, microseconds at context 4096 with 4 warps and the old split count against 8 warps:
        # batch 8 18.8 -> 12.4, batch 16 18.2 -> 15.1, batch 4 12.7 -> 11.3; eight warps want at least 256 keys a block
        # and at most 8 splits: context 1024, batch 8: 2 splits 9.3, 4 splits 8.6; context 4096, batch 1: 8 splits
        # 11.1, 16 splits 12.4)
        # 16 keys per iteration: 160 registers per thread instead of 251, so that a block no longer fills an SM's
        # register file and the product that follows finds room beside it while it waits for it (alone the two variants
        # take the same time; in a 135M decode step: batch 1 0.73 -> 0.65 ms, batch 8 0.80 -> 0.78 ms)
        # (with more than 1,024 keys per block the longer loop of the 16-key variant costs more than the room gains:
        # 360M shapes at batch 8, three splits of 1,365 keys: 1.23 ms with 32 keys per iteration, 1.27 ms with 16)
        splits = max(1, min(148 // pairs, 8, -(-max_context // 256)))
        return splits, (16 if max_context <= 1024 * splits else 0), 8
    return max(1, min(-(-148 // pairs), most)), 0, 4


def decode_mma_splits(n: int, nkv: int, hd: int, max_context: int) -> int:
    return decode_mma_plan(n, nkv, hd, max_context)[0]


def attention_decode_mma(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                         block_tables: torch.Tensor, row_seq: torch.Tensor, positions: torch.Tensor, nh: int, nkv: int,
                         hd: int, page_size: int, scale: float, window: Optional[int], splits: int,
                         part_acc: torch.Tensor, part_ml: torch.Tensor, counters: torch.Tensor,
                         status: torch.Tensor, block_keys: int = 0, warps: int = 4, sink_terms=None) -> None:
    """bfloat16 split-key decode attention on the tensor cores. Scratch: part_acc float32
    [n, nh, warps*splits, hd], part_ml float32 [n, nh, warps*splits, 2], counters int32 [n*nkv], zero on entry
    and left zero. ``warps`` per block: 4, or 8 (head size 64). ``sink_terms`` = (r1, r2, sink, gate), each a float32
    tensor or None as in ``sink_attention_rows``: the softmax then has a distance bias, a sink in its denominator and a
    sigmoid gate on each head's output (the kernel's instantiation for these terms; never part of a decode program)."""
    _cuda(q, out, kcache, vcache, block_tables, row_seq, positions, part_acc, part_ml, counters, status)
    n = q.shape[0]
    assert q.dtype == out.dtype == kcache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    assert part_acc.numel() >= n * nh * warps * splits * hd and part_ml.numel() >= n * nh * warps * splits * 2
    assert counters.numel() >= n * nkv
    prog = _program_for(status)
    if sink_terms is not None:
        if prog is not None:
            prog.flush()
        r1, r2, sink, gate = sink_terms
        _cuda(r1, r2, sink, gate)
        _call("gb_attention_decode_mma_sink", _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache),
              _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), _ptr(positions), n, nh, nkv, hd, page_size,
              kcache.shape[0], float(scale), int(window or 0), int(splits), _ptr(part_acc), _ptr(part_ml), _ptr(counters),
              _ptr(status), 1 if USE_PDL else 0, int(block_keys), int(warps), *_sink_args(r1, r2, sink, gate, nh), _stream())
        return
    if prog is not None and prog.takes_rows(n):
        if not prog.takes_attention(hd, block_keys):
            prog.flush()
            prog._status = status
        prog._add("gb_program_encode_attention", splits * nkv * n, n, 8, _ptr(q), q.stride(0), _ptr(out), out.stride(0),
                  _ptr(kcache), _ptr(vcache), _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), _ptr(positions), n,
                  nh, nkv, hd, page_size, kcache.shape[0], float(scale), int(window or 0), int(splits), _ptr(part_acc),
                  _ptr(part_ml), _ptr(counters), _ptr(status), int(block_keys))
        prog._hd, prog._bk = hd, (16 if (hd == 64 and block_keys == 16) or hd == 128 else 32)
        return
    _call("gb_attention_decode_mma_pdl", _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache),
          _ptr(block_tables), block_tables.shape[1], _ptr(row_seq), _ptr(positions), n, nh, nkv, hd, page_size,
          kcache.shape[0], float(scale), int(window or 0), int(splits), _ptr(part_acc), _ptr(part_ml), _ptr(counters),
          _ptr(status), 1 if USE_PDL else 0, int(block_keys), int(warps), _stream())


def attention_prefill_supported(dtype: torch.dtype, nh: int, nkv: int, hd: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib().gb_attention_prefill_supported(nh, nkv, hd, page_size))


def attention_prefill_tc_supported(q: torch.Tensor, out: torch.Tensor, nh: int, nkv: int, hd: int, page_size: int) -> bool:
    """Whether the tcgen05 flash-attention kernel takes these operands (bfloat16, head size 64, rows
    aligned for TMA)."""
    return (q.dtype == torch.bfloat16 and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
            and out.data_ptr() % 16 == 0 and bool(lib().gb_attention_prefill_tc_supported(nh, nkv, hd, page_size)))


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                         block_tables: torch.Tensor, seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor,
                         max_rows_per_seq: int, nh: int, nkv: int, hd: int, page_size: int, scale: float,
                         window: Optional[int], status: torch.Tensor, sink_terms=None) -> None:
    """bfloat16 flash attention on tcgen05 (TMA loads from the paged cache, S and PV in tensor memory) for
    batches whose requests bring runs of consecutive rows; arguments as ``attention_prefill``. ``sink_terms`` =
    (r1, r2, sink, gate), each a float32 tensor or None as in ``sink_attention_rows``: the kernel's instantiation whose
    softmax has a distance bias, a sink in its denominator and a sigmoid gate on each head's output."""
    _cuda(q, out, kcache, vcache, block_tables, seq_first_row, seq_start_pos, status)
    assert q.dtype == out.dtype == kcache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape[1:] == (nkv, page_size, hd)
    S = block_tables.shape[0]
    assert seq_first_row.numel() == S + 1 and seq_start_pos.numel() == S
    if sink_terms is not None:
        r1, r2, sink, gate = sink_terms
        _cuda(r1, r2, sink, gate)
        _call("gb_attention_prefill_tc_sink", _ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), _ptr(kcache),
              _ptr(vcache), _ptr(block_tables), block_tables.shape[1], _ptr(seq_first_row), _ptr(seq_start_pos), S,
              int(max_rows_per_seq), nh, nkv, hd, page_size, kcache.shape[0], float(scale), int(window or 0), _ptr(status),
              *_sink_args(r1, r2, sink, gate, nh), _stream())
        return
    _call("gb_attention_prefill_tc", _ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), _ptr(kcache),
          _ptr(vcache), _ptr(block_tables), block_tables.shape[1], _ptr(seq_first_row), _ptr(seq_start_pos), S,
          int(max_rows_per_seq), nh, nkv, hd, page_size, kcache.shape[0], float(scale), int(window or 0), _ptr(status),
          _stream())


def attention_prefill(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                      block_tables: torch.Tensor, seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor,
                      max_rows_per_seq: int, nh: int, nkv: int, hd: int, page_size: int, scale: float,
                      window: Optional[int], status: torch.Tensor) -> None:
    """bfloat16 flash attention for batches whose requests bring runs of consecutive rows.
    seq_first_row int32 [S+1], seq_start_pos int32 [S]; block_tables int32 [S, max_pages]."""
    _cuda(q, out, kcache, vcache, block_tables, seq_first_row, seq_start_pos, status)
    assert q.dtype == out.dtype == kcache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    S = block_tables.shape[0]
    assert seq_first_row.numel() == S + 1 and seq_start_pos.numel() == S
    _call("gb_attention_prefill", _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache),
          _ptr(block_tables), block_tables.shape[1], _ptr(seq_first_row), _ptr(seq_start_pos), S, int(max_rows_per_seq),
          nh, nkv, hd, page_size, kcache.shape[0], float(scale), int(window or 0), _ptr(status), _stream())


def kv_prefetch(kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor, row_seq: torch.Tensor,
                positions: torch.Tensor, nkv: int, hd: int, page_size: int, window: Optional[int],
                blocks_per_row: int) -> None:
    """Ask the memory system to bring the pages that each row's attention will read into L2."""
    _cuda(kcache, vcache, block_tables, row_seq, positions)
    tile_bytes = page_size * hd * kcache.element_size()
    if tile_bytes % 128:
        return
    _call("gb_kv_prefetch", _ptr(kcache), _ptr(vcache), _ptr(block_tables), block_tables.shape[1], _ptr(row_seq),
          _ptr(positions), positions.shape[0], nkv, page_size, kcache.shape[0], tile_bytes, int(window or 0),
          int(blocks_per_row), _stream())


def stream_marker() -> None:
    """An empty kernel on the current stream: a node of its own in a recorded step (see ``GqaAttention.prefetch``)."""
    _call("gb_stream_marker", _stream())


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           uniform: Optional[torch.Tensor] = None, want_slots: Optional[torch.Tensor] = None,
           state: Optional[torch.Tensor] = None, last_token: Optional[torch.Tensor] = None) -> None:
    """out[r] = argmax(logits[r]) where the row's temperature is <= 0 (or none is given), else a draw from
    softmax(logits[r] / temperature) with a uniform number in [0, 1). Temperature and number come from
    ``temperature[r]`` and ``uniform[r]``, or, for rows with ``want_slots[r] >= 0``, from the request's sampling
    state ``state[want_slots[r]]`` (int32 [slots, 4]: generator state low and high word, temperature bits, unused),
    whose xorshift64* generator the kernel advances by one draw. ``last_token`` (int32 [slots]) receives the chosen
    token of every row that names a slot (see ``resolve_tokens``)."""
    _cuda(logits, out, temperature, uniform, want_slots, state, last_token)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    if want_slots is not None:
        assert want_slots.dtype == torch.int32 and want_slots.numel() >= rows
        assert state is not None and state.dtype == torch.int32 and state.shape[1] == 4 and state.is_contiguous()
    _call("gb_sample", _ptr(logits), logits.stride(0), _ptr(temperature), _ptr(uniform), _ptr(want_slots), _ptr(state),
          state.shape[0] if state is not None else 0, _ptr(last_token), _ptr(out), rows, vocab, _stream())


def resolve_tokens(tokens: torch.Tensor, token_slots: torch.Tensor, last_token: torch.Tensor) -> None:
    """tokens[i] = last_token[token_slots[i]] where token_slots[i] >= 0 (in place): rows whose token is what the sampling
    kernel chose for their request in the step before, which the host had not read yet when it launched this step."""
    _cuda(tokens, token_slots, last_token)
    assert tokens.dtype == token_slots.dtype == last_token.dtype == torch.int32 and token_slots.numel() >= tokens.numel()
    _call("gb_resolve_tokens", _ptr(tokens), _ptr(token_slots), _ptr(last_token), tokens.numel(), last_token.numel(), _stream())


# ------------------------------------------------------------------ branches that are normed before they join the residual
def rmsnorm_add(y: torch.Tensor, gain: torch.Tensor, x: torch.Tensor, eps: float, bias: Optional[torch.Tensor] = None,
                copy: Optional[torch.Tensor] = None) -> None:
    """x[r, :] += gain * y[r, :] / sqrt(mean(y[r, :]^2) + eps); everything float32. ``bias`` (float32 [d]) is added to
    y first (y itself is left as it is); ``copy`` ([n, d], float32 or bfloat16, contiguous) receives the new x."""
    _cuda(y, gain, x, bias, copy)
    n, d = x.shape
    assert y.shape == (n, d) and y.dtype == x.dtype == gain.dtype == torch.float32 and gain.numel() == d
    assert y.stride(1) == 1 and x.stride(1) == 1
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == d)
    assert copy is None or (copy.shape == (n, d) and copy.is_contiguous())
    _call("gb_rmsnorm_add", _ptr(y), y.stride(0), _ptr(gain), _ptr(x), x.stride(0), n, d, float(eps), _ptr(bias), _ptr(copy),
          _dt(copy) if copy is not None else 0, _stream())


def cast_rows(x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = x[rows[r], :] (all rows in order, if ``rows`` is None): float32 rows in ``out``'s dtype, rounded once."""
    _cuda(x, out, rows)
    n, d = out.shape
    assert x.dtype == torch.float32 and x.shape[1] == d and x.stride(1) == 1 and out.is_contiguous()
    assert (rows is None and x.shape[0] >= n) or (rows is not None and rows.dtype == torch.int32 and rows.numel() >= n)
    _call("gb_cast_rows", _ptr(x), x.stride(0), _ptr(rows), _ptr(out), _dt(out), n, d, _stream())


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> None:
    """y[r, :] += bias; float32."""
    _cuda(y, bias)
    n, d = y.shape
    assert y.dtype == bias.dtype == torch.float32 and bias.numel() == d and y.stride(1) == 1
    _call("gb_add_bias", _ptr(y), y.stride(0), _ptr(bias), n, d, _stream())


def clamped_glu(gate_up: torch.Tensor, bias: Optional[torch.Tensor], limit: float, slope: float, act: torch.Tensor) -> None:
    """act[r, f] = g * sigmoid(slope * g) * (u + 1) with g = min(gate_up[r, f] + bias[f], limit) and u = clamp(gate_up[r, ff + f]
    + bias[ff + f], -limit, limit), formed in float32; ``gate_up`` [n, 2 ff] float32 or bfloat16, ``bias`` float32 [2 ff] or None."""
    _cuda(gate_up, bias, act)
    n, ff = act.shape
    assert gate_up.shape == (n, 2 * ff) and gate_up.stride(1) == 1 and act.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == 2 * ff)
    _call("gb_clamped_glu", _ptr(gate_up), _dt(gate_up), gate_up.stride(0), _ptr(bias), float(limit), float(slope), _ptr(act), _dt(act),
          n, ff, _stream())


def relu2(h: torch.Tensor, out: torch.Tensor) -> None:
    """out = max(h, 0)^2, element by element."""
    _cuda(h, out)
    assert h.shape == out.shape and h.dtype == out.dtype and h.is_contiguous() and out.is_contiguous()
    _call("gb_relu2", _ptr(h), _ptr(out), _dt(out), h.numel(), _stream())


def scale_(t: torch.Tensor, s: float) -> None:
    """t *= s in place (float32)."""
    _cuda(t)
    assert t.dtype == torch.float32 and t.is_contiguous()
    _call("gb_scale", _ptr(t), t.numel(), float(s), _stream())


def gated_head_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, heads: int, eps: float,
                    gate_silu: bool = False) -> None:
    """out[r, h, :] = weight * o[r, h, :] / sqrt(mean(o[r, h, :]^2) + eps) * sigmoid(gate[r, h, :]); o, gate, weight
    float32 (gate may be a column slice of a wider tensor)."""
    _cuda(o, gate, weight, out)
    n, hv = o.shape
    v = hv // heads
    assert o.dtype == gate.dtype == weight.dtype == torch.float32 and o.is_contiguous() and out.is_contiguous()
    assert gate.shape == (n, hv) and gate.stride(1) == 1 and out.shape == (n, hv) and weight.numel() == v
    _call("gb_gated_head_norm", _ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), _ptr(out), _dt(out), n, heads, v, float(eps),
          1 if gate_silu else 0, _stream())


def gelu_glu(gate_up: torch.Tensor, act: torch.Tensor) -> None:
    """act[r, f] = gelu_tanh(gate_up[r, f]) * gate_up[r, ff + f], the tanh form of GELU on the gate half; float32 arithmetic."""
    _cuda(gate_up, act)
    n, ff = act.shape
    assert gate_up.shape == (n, 2 * ff) and gate_up.stride(1) == 1 and act.is_contiguous()
    _call("gb_gelu_glu", _ptr(gate_up), _dt(gate_up), gate_up.stride(0), _ptr(act), _dt(act), n, ff, _stream())


def scaled_sum(x: torch.Tensor, y: torch.Tensor, a: float, b: float, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (+)= a * x + b * y; float32, same shapes, contiguous."""
    _cuda(x, y, out)
    assert x.dtype == y.dtype == out.dtype == torch.float32 and x.shape == y.shape == out.shape
    assert x.is_contiguous() and y.is_contiguous() and out.is_contiguous()
    _call("gb_scaled_sum", _ptr(x), _ptr(y), float(a), float(b), _ptr(out), x.numel(), 1 if accumulate else 0, _stream())


# ------------------------------------------------------------------------------- attention over a latent cache
def latent_kv_write(proj: torch.Tensor, kv_col: int, qabs: torch.Tensor, cache: torch.Tensor, latent_gain: Optional[torch.Tensor],
                    inv_freq: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, heads: int, dq: int, r: int, c: int,
                    rot_dims: int, eps: float, write_kv: bool, status: torch.Tensor) -> None:
    """Rotate every head's rotated query part of ``proj`` [n, >= heads * (dq + r)] into ``qabs`` [n, heads, c + r][..., c:];
    with ``write_kv`` also RMS-norm the raw latent (columns kv_col .. kv_col + c), rotate the raw shared key part behind it
    and store both at each row's slot of ``cache`` [pages, 1, page_size, c + r]."""
    _cuda(proj, qabs, cache, latent_gain, inv_freq, positions, slots, status)
    n = proj.shape[0]
    assert proj.stride(1) == 1 and qabs.is_contiguous() and cache.is_contiguous() and proj.dtype == qabs.dtype == cache.dtype
    assert qabs.shape[0] == n and qabs.numel() == n * heads * (c + r) and cache.shape[-1] == c + r
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() >= rot_dims // 2
    num_slots = cache.numel() // (c + r)
    _call("gb_latent_kv_write", _ptr(proj), proj.stride(0), kv_col, _ptr(qabs), _ptr(cache), _dt(proj), _ptr(latent_gain),
          _ptr(inv_freq), _ptr(positions), _ptr(slots), n, heads, dq, r, c, rot_dims, num_slots, float(eps),
          1 if write_kv else 0, _ptr(status), _stream())


def latent_attention_rows(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                          row_seq: torch.Tensor, positions: torch.Tensor, sink: Optional[torch.Tensor], heads: int, c: int, r: int,
                          page_size: int, scale: float, window: Optional[int], status: torch.Tensor) -> None:
    """out[row, head, :c] = sum_j p_j latent_j with p the softmax (with an optional sink logit per head in the denominator)
    of scale * q[row, head, :] . cache_row_j over the row's visible tokens; one warp per (row, head), float32 arithmetic."""
    _cuda(q, out, cache, block_tables, row_seq, positions, sink, status)
    n = q.shape[0]
    assert q.is_contiguous() and out.is_contiguous() and cache.is_contiguous() and q.dtype == out.dtype == cache.dtype
    assert q.numel() == n * heads * (c + r) and out.numel() == n * heads * c and cache.shape[-1] == c + r
    num_pages = cache.numel() // ((c + r) * page_size)
    _call("gb_latent_attention_rows", _ptr(q), _ptr(out), _dt(q), _ptr(cache), _ptr(block_tables), block_tables.shape[1],
          _ptr(row_seq), _ptr(positions), _ptr(sink), n, heads, c, r, page_size, num_pages, float(scale),
          int(window) if window else 0, _ptr(status), _stream())


def head_linear_supported(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, a_head: int, c_head: int) -> bool:
    """Whether ``head_linear`` takes these operands: bfloat16, a head's input size a multiple of 16 up to 256, aligned."""
    if not (a.dtype == w.dtype == out.dtype == torch.bfloat16) or w.dim() != 3 or not w.is_contiguous():
        return False
    if a.stride(1) != 1 or out.stride(1) != 1:
        return False
    return bool(lib().gb_head_linear_supported(_ptr(a), a.stride(0), a_head, _ptr(w), _ptr(out), out.stride(0), c_head,
                                               w.shape[1], w.shape[2]))


def head_linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, a_head: int, c_head: int) -> None:
    """out[row, h * c_head : h * c_head + N] = a[row, h * a_head : h * a_head + K] @ w[h]^T for every head h of
    w [heads, N, K], in one launch (bfloat16, float32 sums)."""
    _cuda(a, w, out)
    heads, N, K = w.shape
    n = a.shape[0]
    assert out.shape[0] == n and a.shape[1] >= (heads - 1) * a_head + K and out.shape[1] >= (heads - 1) * c_head + N
    _call("gb_head_linear", _ptr(a), a.stride(0), a_head, _ptr(w), _ptr(out), out.stride(0), c_head, n, heads, N, K, _stream())


def latent_attention_mma_supported(dtype: torch.dtype, c: int, r: int, page_size: int) -> bool:
    """Whether the tensor-core kernel takes this latent size, rotated size and page size (bfloat16 only)."""
    return dtype == torch.bfloat16 and bool(lib().gb_latent_attention_mma_supported(c, r, page_size))


def latent_decode_splits(num_seqs: int, heads: int, max_context: int, target_blocks: int = 148 * 5) -> int:
    """Into how many shares the keys of a decoded row are cut: blocks are (share, group of 16 heads, request), a share is
    at least one tile of 64 keys, and a block keeps only one tile's load in flight while it works on another, so it
    takes about five resident blocks per SM (what their shared memory allows) to keep the memory system busy."""
    blocks = max(num_seqs, 1) * -(-heads // 16)
    tiles = max(1, -(-max_context // 64))
    return max(1, min(tiles, -(-target_blocks // blocks), 64))


def latent_attention_mma(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                         seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor, positions: torch.Tensor,
                         sink: Optional[torch.Tensor], heads: int, c: int, r: int, page_size: int, scale: float,
                         window: Optional[int], status: torch.Tensor, *, max_rows_per_seq: int = 0, decode: bool = False,
                         splits: int = 1, part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None) -> None:
    """As ``latent_attention_rows`` on the tensor cores, heads packed into the tiles' rows. ``decode``: every request of the
    step brings one row (row i is request i) and its keys are cut into ``splits`` shares (``part_o`` float32
    [n, heads * splits * c] and ``part_ml`` [n, heads * splits * 2] when more than one); otherwise the step's requests
    bring runs of rows, none longer than ``max_rows_per_seq``."""
    _cuda(q, out, cache, block_tables, seq_first_row, seq_start_pos, positions, sink, status, part_o, part_ml)
    n = q.shape[0]
    assert q.dtype == out.dtype == cache.dtype == torch.bfloat16 and q.is_contiguous() and out.is_contiguous() and cache.is_contiguous()
    assert q.numel() == n * heads * (c + r) and out.numel() == n * heads * c and cache.shape[-1] == c + r
    S = seq_start_pos.shape[0]
    if decode:
        assert S == n
        if splits > 1:
            assert part_o.dtype == part_ml.dtype == torch.float32 and part_o.numel() >= n * heads * splits * c
            assert part_ml.numel() >= n * heads * splits * 2
    num_pages = cache.numel() // ((c + r) * page_size)
    _call("gb_latent_attention_mma", _ptr(q), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(cache), _ptr(block_tables),
          block_tables.shape[1], _ptr(seq_first_row), _ptr(seq_start_pos), _ptr(positions), _ptr(sink), n, S,
          int(max_rows_per_seq), heads, c, r, page_size, num_pages, float(scale), int(window) if window else 0,
          1 if decode else 0, int(splits), _ptr(status), _stream())


# ------------------------------------------------------------------------------------- recurrent state mixers
def short_conv(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, state: torch.Tensor, state_off: int, ctx_row_seq: torch.Tensor,
               positions: torch.Tensor, seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor, seq_slots: torch.Tensor,
               update_state: bool, status: torch.Tensor) -> None:
    """y[t, c] = silu(sum_j w[c, j] * x[t - (taps - 1) + j, c]) along each request's rows; inputs from before the step come
    from (and, with ``update_state``, the last taps - 1 inputs go to) the request's slot of ``state`` [slots, numbers],
    at ``state_off``, laid out [taps - 1, channels]. x may be a column slice; float32."""
    _cuda(x, w, y, state, ctx_row_seq, positions, seq_first_row, seq_start_pos, seq_slots, status)
    n, C = y.shape
    taps = w.shape[1]
    assert x.shape == (n, C) and x.stride(1) == 1 and y.stride(1) == 1 and w.shape == (C, taps) and w.is_contiguous()
    assert x.dtype == y.dtype == w.dtype == state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous()
    assert state_off + (taps - 1) * C <= state.shape[1]
    _call("gb_short_conv", _ptr(x), x.stride(0), _ptr(w), _ptr(y), y.stride(0), _ptr(state), state.stride(0), state_off,
          _ptr(ctx_row_seq), _ptr(positions), _ptr(seq_first_row), _ptr(seq_start_pos), _ptr(seq_slots), n, seq_start_pos.shape[0],
          C, taps, state.shape[0], 1 if update_state else 0, _ptr(status), _stream())


def channel_delta(qkv: torch.Tensor, beta: torch.Tensor, a: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
                  state: torch.Tensor, out: torch.Tensor, seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor,
                  seq_slots: torch.Tensor, heads: int, kv_heads: int, dk: int, dv: int, write_state: bool,
                  status: torch.Tensor, decay_per_head: bool = False) -> None:
    """The gated delta rule, token by token along each request's rows, from and to the request's slot of ``state`` [slots,
    numbers] (S = [heads, dk, dv] first). qkv float32 [n, 2 * kv_heads * dk + heads * dv] (q, k, v after their
    convolutions), beta [n, heads] logits, a the decay's logits: [n, heads * dk] with ``dt_bias`` [heads * dk] (a decay per
    head and key channel) or, with ``decay_per_head``, [n, heads] and [heads] (column slices allowed); out float32
    [n, heads * dv] is the read-out before its norm."""
    _cuda(qkv, beta, a, dt_bias, a_log, state, out, seq_first_row, seq_start_pos, seq_slots, status)
    n = qkv.shape[0]
    dc = 1 if decay_per_head else dk
    for t in (qkv, beta, a, dt_bias, a_log, state, out):
        assert t.dtype == torch.float32
    assert qkv.shape[1] == 2 * kv_heads * dk + heads * dv and qkv.stride(1) == 1 and beta.shape == (n, heads)
    assert a.shape == (n, heads * dc) and a.stride(1) == 1 and beta.stride(1) == 1 and out.shape == (n, heads * dv)
    assert out.is_contiguous() and state.dim() == 2 and state.is_contiguous() and state.shape[1] >= heads * dk * dv
    assert dt_bias.numel() == heads * dc and a_log.numel() == heads
    _call("gb_channel_delta", _ptr(qkv), qkv.stride(0), _ptr(beta), beta.stride(0), _ptr(a), a.stride(0), _ptr(dt_bias),
          _ptr(a_log), _ptr(state), state.stride(0), _ptr(out), _ptr(seq_first_row), _ptr(seq_start_pos), _ptr(seq_slots),
          seq_start_pos.shape[0], heads, kv_heads, dk, dv, state.shape[0], 1 if write_state else 0, _ptr(status), dc, 0, _stream())


CD_SILU_INPUTS, CD_PLAIN, CD_GATE_SILU, CD_NO_NORM = 1, 2, 4, 8


def decay_linear_attention(qkv: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, out: torch.Tensor, seq_first_row: torch.Tensor,
                           seq_start_pos: torch.Tensor, seq_slots: torch.Tensor, heads: int, dk: int, dv: int, write_state: bool,
                           status: torch.Tensor, silu_inputs: bool = True) -> None:
    """Linear attention with a fixed decay per head, token by token along each request's rows, on the delta rule's kernel
    with the correction switched off: S <- decay_h S + k v^T, o = S^T q, S float32 [heads, dk, dv] at the start of the
    request's slot of ``state``. qkv float32 [n, 2 * heads * dk + heads * dv] (column slice allowed); with ``silu_inputs``
    q, k and v pass SiLU as they are read. decay float32 [heads]; out float32 [n, heads * dv]."""
    _cuda(qkv, decay, state, out, seq_first_row, seq_start_pos, seq_slots, status)
    n = qkv.shape[0]
    for t in (qkv, decay, state, out):
        assert t.dtype == torch.float32
    assert qkv.shape[1] == 2 * heads * dk + heads * dv and qkv.stride(1) == 1 and out.shape == (n, heads * dv) and out.is_contiguous()
    assert state.dim() == 2 and state.is_contiguous() and state.shape[1] >= heads * dk * dv and decay.numel() == heads
    _call("gb_channel_delta", _ptr(qkv), qkv.stride(0), 0, 0, 0, 0, 0, _ptr(decay), _ptr(state), state.stride(0), _ptr(out),
          _ptr(seq_first_row), _ptr(seq_start_pos), _ptr(seq_slots), seq_start_pos.shape[0], heads, heads, dk, dv, state.shape[0],
          1 if write_state else 0, _ptr(status), 1, CD_PLAIN | (CD_SILU_INPUTS if silu_inputs else 0), _stream())


#: fewest rows of a piece when a long portion of linear attention with a fixed decay is cut up, and from how many rows on it is
LINEAR_PIECE_ROWS, LINEAR_PIECES_FROM = 128, 384


def linear_piece_rows(longest: int, heads: int, dk: int, dv: int) -> int:
    """Rows of a piece for a step whose longest portion has ``longest`` rows, or 0 where the portion is too short to cut.
    Short pieces are as good as long ones: the walking kernel is bound by what a multiprocessor issues as much as by the
    chain (two of its blocks on one multiprocessor take nearly twice as long), so what the pieces buy is the multiprocessors
    that one walk leaves idle. Measured alone at 8 heads x 128 x 128, 2,048 rows: one walk 690 us, pieces of 128 rows 396 us,
    of 512 rows 539 us; at 16 heads (128 blocks a walk) one walk 718-736 us, pieces of 128 rows 838 us, of 1,024 rows 1,075 us;
    inside a model's prompt step the pieces of 128 are the faster form at both sizes (7.86 against 9.65 ms at 8 heads, 15.0
    against 15.3 ms at 16)."""
    return LINEAR_PIECE_ROWS if longest >= LINEAR_PIECES_FROM else 0


def linear_pieces_needed(n: int, num_seqs: int, piece_rows: int = LINEAR_PIECE_ROWS) -> int:
    """How many pieces ``decay_linear_attention_pieces`` may need for a step of ``n`` rows in ``num_seqs`` sequences."""
    return n // piece_rows + num_seqs


def decay_linear_attention_pieces(qkv: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, out: torch.Tensor, seq_first_row: torch.Tensor,
                                  seq_start_pos: torch.Tensor, seq_slots: torch.Tensor, heads: int, dk: int, dv: int, write_state: bool,
                                  status: torch.Tensor, meta: torch.Tensor, piece_state: torch.Tensor, silu_inputs: bool = True,
                                  piece_rows: int = LINEAR_PIECE_ROWS) -> None:
    """``decay_linear_attention`` with every request's rows cut into pieces of ``piece_rows`` that walk side by side from a
    zero state; the pieces' states are then chained and q^T S_start is added to every read-out. The same sums in another
    order: the chain of dependent updates is one piece long. ``meta`` int32 [4 * P + 2 * num_seqs + 1] and ``piece_state`` float32
    [P, heads * dk * dv] are scratch, P = ``linear_pieces_needed``."""
    _cuda(qkv, decay, state, out, seq_first_row, seq_start_pos, seq_slots, status, meta, piece_state)
    n, S = qkv.shape[0], seq_start_pos.shape[0]
    P = piece_state.shape[0]
    for t in (qkv, decay, state, out, piece_state):
        assert t.dtype == torch.float32
    assert qkv.shape[1] == 2 * heads * dk + heads * dv and qkv.stride(1) == 1 and out.shape == (n, heads * dv) and out.is_contiguous()
    assert state.dim() == 2 and state.is_contiguous() and state.shape[1] >= heads * dk * dv and decay.numel() == heads
    assert P >= linear_pieces_needed(n, S, piece_rows) and piece_state.shape[1] == heads * dk * dv and piece_state.is_contiguous()
    assert meta.dtype == torch.int32 and meta.numel() >= 4 * P + 2 * S + 1 and meta.is_contiguous()
    _call("gb_decay_linear_pieces", _ptr(qkv), qkv.stride(0), _ptr(decay), _ptr(state), state.stride(0), _ptr(out), _ptr(seq_first_row),
          _ptr(seq_start_pos), _ptr(seq_slots), S, n, heads, dk, dv, state.shape[0], 1 if write_state else 0, _ptr(status),
          1 if silu_inputs else 0, int(piece_rows), P, _ptr(meta), _ptr(piece_state), _stream())


def decay_linear_attention_decode(qkv: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, out: torch.Tensor, seq_first_row: torch.Tensor,
                                  seq_start_pos: torch.Tensor, seq_slots: torch.Tensor, heads: int, dk: int, dv: int, write_state: bool,
                                  status: torch.Tensor, silu_inputs: bool = True) -> None:
    """``decay_linear_attention`` for a step in which every request brings one row, on the delta rule's decoding form (S read and
    written once, in whole rows); key and value size up to 128. out float32 [n, heads * dv]: the read-out as it is."""
    _cuda(qkv, decay, state, out, seq_first_row, seq_start_pos, seq_slots, status)
    n = qkv.shape[0]
    for t in (qkv, decay, state, out):
        assert t.dtype == torch.float32
    assert qkv.shape[1] == 2 * heads * dk + heads * dv and qkv.stride(1) == 1 and out.shape == (n, heads * dv) and out.is_contiguous()
    assert state.dim() == 2 and state.is_contiguous() and state.shape[1] >= heads * dk * dv and decay.numel() == heads
    _call("gb_channel_delta_decode", _ptr(qkv), qkv.stride(0), 0, 0, 0, 0, 0, _ptr(decay), _ptr(state), state.stride(0), 0, 0, 0, 0.0,
          _ptr(out), F32, _ptr(seq_first_row), _ptr(seq_start_pos), _ptr(seq_slots), seq_start_pos.shape[0], heads, heads, dk, dv,
          state.shape[0], 1 if write_state else 0, _ptr(status), 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1,
          CD_PLAIN | CD_NO_NORM | (CD_SILU_INPUTS if silu_inputs else 0), _stream())


def residual_conv(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, state: torch.Tensor, state_off: int, row_seq: torch.Tensor,
                  positions: torch.Tensor, seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor, seq_slots: torch.Tensor,
                  update_state: bool, status: torch.Tensor, single_rows: bool = False) -> None:
    """y[t, c] = x[t, c] + sum_j w[c, j] * x[t - (taps - 1) + j, c] along each request's rows (x, y [n, C] in the activation
    dtype, different buffers; sums in float32). Inputs from before the step come from (and, with ``update_state``, the last
    taps - 1 inputs go to) the request's slot of ``state`` float32 [slots, numbers], at ``state_off``, laid out [taps - 1, C].
    ``single_rows``: every request brings exactly one row; the last inputs are then moved up by the same launch."""
    _cuda(x, w, y, state, row_seq, positions, seq_first_row, seq_start_pos, seq_slots, status)
    n, C = x.shape
    taps = w.shape[1]
    assert y.shape == (n, C) and x.is_contiguous() and y.is_contiguous() and x.dtype == y.dtype and w.shape == (C, taps) and w.is_contiguous()
    assert x.data_ptr() != y.data_ptr() and state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous()
    assert state_off + (taps - 1) * C <= state.shape[1]
    _call("gb_residual_conv", _ptr(x), _dt(x), _ptr(w), _dt(w), _ptr(y), _ptr(state), state.stride(0), state_off, _ptr(row_seq),
          _ptr(positions), _ptr(seq_first_row), _ptr(seq_start_pos), _ptr(seq_slots), n, seq_start_pos.shape[0], C, taps, state.shape[0],
          (2 if single_rows else 1) if update_state else 0, _ptr(status), _stream())


def channel_delta_decode_supported(dk: int, dv: int) -> bool:
    return bool(lib().gb_channel_delta_decode_supported(dk, dv))


class DeltaDecodeFusion:
    """What the fused decoding form of the delta rule reads instead of finished q, k, v, decay and gate logits: the stacked
    projection's raw rows ``proj`` float32 [n, >= conv channels + ranks] (q | k | v channels before their convolutions; at
    column ``a1_at`` the low-rank input of the decay, ``w_a2.shape[1]`` numbers, then that of the gate), the convolutions'
    weights [channels, taps] and where in a slot their last inputs start, and the two second-level matrices."""
    __slots__ = ("proj", "conv_w", "conv_state_off", "a1_at", "w_a2", "w_g2")

    def __init__(self, proj, conv_w, conv_state_off, a1_at, w_a2, w_g2):
        self.proj, self.conv_w, self.conv_state_off, self.a1_at, self.w_a2, self.w_g2 = proj, conv_w, conv_state_off, a1_at, w_a2, w_g2

    @staticmethod
    def supported(w_a2: torch.Tensor, w_g2: torch.Tensor) -> bool:
        return (w_a2.dtype == w_g2.dtype and w_a2.dtype in _DT and w_a2.is_contiguous() and w_g2.is_contiguous()
                and w_a2.shape[1] + w_g2.shape[1] <= 512)


def channel_delta_decode(qkv: Optional[torch.Tensor], beta: torch.Tensor, a: Optional[torch.Tensor], dt_bias: torch.Tensor,
                         a_log: torch.Tensor, state: torch.Tensor, gate: Optional[torch.Tensor], norm_weight: torch.Tensor,
                         eps: float, att: torch.Tensor, seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor,
                         seq_slots: torch.Tensor, heads: int, kv_heads: int, dk: int, dv: int, write_state: bool,
                         status: torch.Tensor, fusion: Optional[DeltaDecodeFusion] = None, decay_per_head: bool = False,
                         gate_silu: bool = False) -> None:
    """``channel_delta`` for a step in which every request brings one row, with the read-out's norm and gate applied as
    well: ``att`` [n, heads * dv] (any activation dtype) = norm_weight * o / rms(o) * sigmoid(gate). Reads and writes
    each request's S once, in whole rows. With ``fusion`` the kernel also computes the convolutions of q, k, v (reading
    the slot's last inputs; ``short_conv_state`` must shift them afterwards) and the two low-rank products itself:
    ``qkv``, ``a`` and ``gate`` are then None."""
    _cuda(qkv, beta, a, dt_bias, a_log, state, gate, norm_weight, att, seq_first_row, seq_start_pos, seq_slots, status)
    n = beta.shape[0]
    for t in (beta, dt_bias, a_log, state, norm_weight):
        assert t.dtype == torch.float32
    assert beta.shape == (n, heads) and beta.stride(1) == 1 and att.shape == (n, heads * dv) and att.is_contiguous()
    assert state.dim() == 2 and state.is_contiguous() and state.shape[1] >= heads * dk * dv and norm_weight.numel() == dv
    if fusion is None:
        for t in (qkv, a, gate):
            assert t.dtype == torch.float32 and t.stride(1) == 1
        assert qkv.shape == (n, 2 * kv_heads * dk + heads * dv) and gate.shape == (n, heads * dv)
        assert a.shape == (n, heads * (1 if decay_per_head else dk)) and dt_bias.numel() == a.shape[1]
        extra = (0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0)
        ptrs = (_ptr(qkv), qkv.stride(0), _ptr(a), a.stride(0), _ptr(gate), gate.stride(0))
    else:
        f = fusion
        _cuda(f.proj, f.conv_w, f.w_a2, f.w_g2)
        channels = 2 * kv_heads * dk + heads * dv
        ra, rg = f.w_a2.shape[1], f.w_g2.shape[1]
        taps = f.conv_w.shape[1]
        assert DeltaDecodeFusion.supported(f.w_a2, f.w_g2) and f.proj.dtype == f.conv_w.dtype == torch.float32
        assert f.proj.shape[0] == n and f.proj.stride(1) == 1 and f.proj.shape[1] >= f.a1_at + ra + rg and f.a1_at >= channels
        assert f.conv_w.shape == (channels, taps) and f.conv_w.is_contiguous()
        assert f.w_a2.shape[0] == heads * dk and f.w_g2.shape[0] == heads * dv
        assert f.conv_state_off + (taps - 1) * channels <= state.shape[1]
        extra = (_ptr(f.proj), f.proj.stride(0), _ptr(f.conv_w), f.conv_state_off, taps, f.a1_at, ra, rg, _ptr(f.w_a2), _ptr(f.w_g2),
                 _dt(f.w_a2))
        ptrs = (0, 0, 0, 0, 0, 0)
    _call("gb_channel_delta_decode", ptrs[0], ptrs[1], _ptr(beta), beta.stride(0), ptrs[2], ptrs[3], _ptr(dt_bias),
          _ptr(a_log), _ptr(state), state.stride(0), ptrs[4], ptrs[5], _ptr(norm_weight), float(eps), _ptr(att),
          _dt(att), _ptr(seq_first_row), _ptr(seq_start_pos), _ptr(seq_slots), seq_start_pos.shape[0], heads, kv_heads, dk, dv,
          state.shape[0], 1 if write_state else 0, _ptr(status), *extra, 1 if decay_per_head else dk,
          CD_GATE_SILU if gate_silu else 0, _stream())


def short_conv_state(x: torch.Tensor, state: torch.Tensor, state_off: int, taps: int, seq_first_row: torch.Tensor,
                     seq_start_pos: torch.Tensor, seq_slots: torch.Tensor) -> None:
    """The second half of ``short_conv`` alone: each request's slot keeps the last taps - 1 rows of ``x`` [n, channels]
    (shifting in what it held when the request brings fewer rows)."""
    _cuda(x, state, seq_first_row, seq_start_pos, seq_slots)
    n, C = x.shape
    assert x.dtype == state.dtype == torch.float32 and x.stride(1) == 1 and state.dim() == 2 and state.is_contiguous()
    assert state_off + (taps - 1) * C <= state.shape[1]
    _call("gb_short_conv_state", _ptr(x), x.stride(0), _ptr(state), state.stride(0), state_off, _ptr(seq_first_row),
          _ptr(seq_start_pos), _ptr(seq_slots), seq_start_pos.shape[0], C, taps, state.shape[0], _stream())


# ------------------------------------------------------------------- layer norm and a residual kept as several streams
def streams_broadcast(x: torch.Tensor, xs: torch.Tensor, streams: int) -> None:
    """xs[r, s, :] = x[r, :] for every stream s; float32."""
    _cuda(x, xs)
    n, d = x.shape
    assert x.dtype == xs.dtype == torch.float32 and x.is_contiguous() and xs.is_contiguous() and xs.shape == (n, streams * d)
    _call("gb_streams_broadcast", _ptr(x), _ptr(xs), n, streams, d, _stream())


class WeightedRows:
    """A branch output that exists only as its parts: y[r] = sum_k weight[r, k] * pair[r, k, :] + gate[r] * shared[r, :]
    (``shared`` and ``gate`` optional; without a gate the shared row is added as it is). ``streams_step`` takes it in the
    place of a stored y and forms the sum on the way."""
    __slots__ = ("pair", "weight", "shared", "gate")

    def __init__(self, pair: torch.Tensor, weight: torch.Tensor, shared: Optional[torch.Tensor] = None,
                 gate: Optional[torch.Tensor] = None):
        self.pair, self.weight, self.shared, self.gate = pair, weight, shared, gate


def streams_step(xs: torch.Tensor, streams: int, *, fold=None, read: Optional[torch.Tensor] = None, norm=None,
                 h: Optional[torch.Tensor] = None, u_out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                 positions: Optional[torch.Tensor] = None) -> None:
    """One pass over the rows of a residual kept as ``streams`` rows per token (xs float32 [n, streams * d]; one stream: the
    plain residual). ``fold`` = (y, mix, write): first x_t <- sum_s mix[s, t] x_s + write[t] * y for all streams at once (y
    float32 [n, d], or a ``WeightedRows``; stored back unless ``rows`` gathers). Then u = sum_s read[s] x_s (``read`` None:
    the plain sum), stored as float32 into ``u_out`` and / or through the layer norm ``norm`` = (weight, bias or None, eps)
    into ``h`` (any activation dtype). ``rows`` (int32) picks the input row of each output row; ``positions`` marks padding
    rows (< 0), which are skipped."""
    _cuda(xs, read, h, u_out, rows, positions)
    n_src = xs.shape[0]
    d = xs.shape[1] // streams
    assert xs.dtype == torch.float32 and xs.is_contiguous() and xs.shape[1] == streams * d
    n_out = rows.shape[0] if rows is not None else n_src
    y = mix = write = lazy = None
    if fold is not None:
        y, mix, write = fold
        if isinstance(y, WeightedRows):
            lazy, y = y, None
            top = lazy.weight.shape[1]
            _cuda(lazy.pair, lazy.weight, lazy.shared, lazy.gate)
            assert lazy.pair.dtype == lazy.weight.dtype == torch.float32 and lazy.pair.shape == (n_src, top * d)
            assert lazy.pair.is_contiguous() and lazy.weight.is_contiguous() and lazy.weight.shape[0] == n_src
            assert lazy.shared is None or (lazy.shared.dtype == torch.float32 and lazy.shared.shape == (n_src, d) and lazy.shared.stride(1) == 1)
            assert lazy.gate is None or (lazy.gate.dtype == torch.float32 and lazy.gate.numel() >= n_src)
        else:
            assert y.dtype == torch.float32 and y.shape == (n_src, d) and y.stride(1) == 1
        assert mix.dtype == write.dtype == torch.float32
        assert mix.numel() == streams * streams and write.numel() == streams and mix.is_contiguous()
    w = b = None
    eps = 0.0
    if h is not None:
        w, b, eps = norm
        assert h.shape == (n_out, d) and h.is_contiguous() and w.dtype == torch.float32 and w.numel() == d
        assert b is None or (b.dtype == torch.float32 and b.numel() == d)
    assert read is None or (read.dtype == torch.float32 and read.numel() == streams)
    assert u_out is None or (u_out.dtype == torch.float32 and u_out.shape == (n_out, d) and u_out.is_contiguous())
    _call("gb_streams_step", _ptr(xs), streams, d, _ptr(y), y.stride(0) if y is not None else 0,
          _ptr(lazy.pair) if lazy else 0, _ptr(lazy.weight) if lazy else 0, lazy.weight.shape[1] if lazy else 0,
          _ptr(lazy.shared) if lazy else 0, lazy.shared.stride(0) if lazy and lazy.shared is not None else 0,
          _ptr(lazy.gate) if lazy else 0, _ptr(mix), _ptr(write), _ptr(read),
          _ptr(w), _ptr(b), float(eps), _ptr(h), _dt(h) if h is not None else F32, _ptr(u_out), _ptr(rows), _ptr(positions),
          n_out, n_src, _stream())


# ------------------------------------------------------------------------------------ attention without a softmax
def qk_norm_rope_write(qkv: torch.Tensor, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                       positions: torch.Tensor, slots: torch.Tensor, q_out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                       heads: int, kv_heads: int, dim: int, vdim: int, rot: int, eps: float, page_size: int, write_kv: bool,
                       status: torch.Tensor, values_out: Optional[torch.Tensor] = None, values_in: Optional[torch.Tensor] = None,
                       value_mix: Optional[torch.Tensor] = None) -> None:
    """From the float32 sums of the stacked projection q | k | v: RMS norm of every query and key head over ``dim`` (one
    gain for the query heads, one for the key heads; None: no norm), rotation of the first ``rot`` channels in neighbouring pairs by
    float32(position) * inv_freq[i], q into ``q_out`` [n, heads * dim], k and v into the paged cache at each row's slot.
    With ``values_in`` (float32 [n, kv_heads * vdim]) a row's v becomes (1 - value_mix) v + value_mix values_in[row] first
    (``value_mix`` one float32 number on the device); ``values_out`` (same shape) receives the row's v as it is stored."""
    _cuda(qkv, q_gain, k_gain, inv_freq, positions, slots, q_out, kcache, vcache, status, values_out, values_in, value_mix)
    for t in (values_out, values_in):
        assert t is None or (t.dtype == torch.float32 and t.shape == (qkv.shape[0], kv_heads * vdim) and t.stride(1) == 1)
    assert values_out is None or values_in is None or values_out.stride(0) == values_in.stride(0)
    assert values_in is None or (value_mix is not None and value_mix.dtype == torch.float32 and value_mix.numel() == 1)
    ld_values = (values_out if values_out is not None else values_in).stride(0) if (values_out is not None or values_in is not None) else 0
    n = qkv.shape[0]
    assert qkv.dtype == torch.float32 and qkv.stride(1) == 1 and qkv.shape[1] == (heads + kv_heads) * dim + kv_heads * vdim
    for gain in (q_gain, k_gain):
        assert gain is None or (gain.dtype == torch.float32 and gain.numel() == dim)
    assert q_out.shape == (n, heads * dim) and q_out.is_contiguous() and q_out.dtype == kcache.dtype == vcache.dtype
    assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape[-1] == dim and vcache.shape[-1] == vdim
    assert rot == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot // 2)
    _call("gb_qk_norm_rope_write", _ptr(qkv), qkv.stride(0), _ptr(q_gain), _ptr(k_gain), _ptr(inv_freq), _ptr(positions), _ptr(slots),
          _ptr(q_out), _ptr(kcache), _ptr(vcache), _dt(q_out), n, heads, kv_heads, dim, vdim, rot, float(eps), page_size,
          kcache.shape[0] * page_size, 1 if write_kv else 0, _ptr(status), _ptr(values_out), _ptr(values_in), ld_values,
          _ptr(value_mix) if values_in is not None else 0, _stream())


def sigmoid_attention_rows(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                           row_seq: torch.Tensor, positions: torch.Tensor, head_bias: Optional[torch.Tensor], heads: int, kv_heads: int,
                           dim: int, vdim: int, page_size: int, scale: float, window: Optional[int], status: torch.Tensor) -> None:
    """out[row, head, :] = sum over the row's visible keys of sigmoid(q . k * scale + head_bias[head]) * v: no softmax, the
    weights are not normalised over the keys. One warp per (row, head); any row, both dtypes."""
    _cuda(q, out, kcache, vcache, block_tables, row_seq, positions, head_bias, status)
    n = q.shape[0]
    assert q.shape == (n, heads * dim) and out.shape == (n, heads * vdim) and q.is_contiguous() and out.is_contiguous()
    assert q.dtype == out.dtype == kcache.dtype == vcache.dtype and block_tables.is_contiguous()
    assert head_bias is None or (head_bias.dtype == torch.float32 and head_bias.numel() == heads)
    _call("gb_sigmoid_attention_rows", _ptr(q), _ptr(out), _dt(q), _ptr(kcache), _ptr(vcache), _ptr(block_tables),
          block_tables.shape[1], _ptr(row_seq), _ptr(positions), _ptr(head_bias), n, heads, kv_heads, dim, vdim, page_size,
          kcache.shape[0], float(scale), int(window) if window else 0, _ptr(status), _stream())


def sigmoid_attention_decode_supported(dtype: torch.dtype, vdim: int) -> bool:
    return dtype in _DT and bool(lib().gb_sigmoid_attention_decode_supported(vdim * (4 if dtype == torch.float32 else 2)))


def sigmoid_attention_decode(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                             row_seq: torch.Tensor, positions: torch.Tensor, head_bias: Optional[torch.Tensor], heads: int, kv_heads: int,
                             dim: int, vdim: int, page_size: int, scale: float, window: Optional[int], status: torch.Tensor) -> None:
    """``sigmoid_attention_rows`` for single decoded tokens: a block of eight warps per (row, head) that share the row's
    keys and add their partial sums in a fixed order; a value row must be 64, 128, 256 or 512 bytes
    (``sigmoid_attention_decode_supported``)."""
    _cuda(q, out, kcache, vcache, block_tables, row_seq, positions, head_bias, status)
    n = q.shape[0]
    assert q.shape == (n, heads * dim) and out.shape == (n, heads * vdim) and q.is_contiguous() and out.is_contiguous()
    assert q.dtype == out.dtype == kcache.dtype == vcache.dtype and block_tables.is_contiguous()
    assert head_bias is None or (head_bias.dtype == torch.float32 and head_bias.numel() == heads)
    _call("gb_sigmoid_attention_decode", _ptr(q), _ptr(out), _dt(q), _ptr(kcache), _ptr(vcache), _ptr(block_tables),
          block_tables.shape[1], _ptr(row_seq), _ptr(positions), _ptr(head_bias), n, heads, kv_heads, dim, vdim, page_size,
          kcache.shape[0], float(scale), int(window) if window else 0, _ptr(status), _stream())


def sigmoid_attention_tiles_supported(dtype: torch.dtype, dim: int, vdim: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib().gb_sigmoid_attention_tiles_supported(dim, vdim))


def sigmoid_attention_tiles(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                            seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor, max_rows_per_seq: int,
                            head_bias: Optional[torch.Tensor], heads: int, kv_heads: int, dim: int, vdim: int, page_size: int,
                            scale: float, window: Optional[int], status: torch.Tensor) -> None:
    """``sigmoid_attention_rows`` for runs of consecutive rows (prompt portions) in bfloat16 on the tensor cores: a block
    takes 64 rows of one request and one head; ``max_rows_per_seq`` bounds the rows a request brings (it sizes the grid)."""
    _cuda(q, out, kcache, vcache, block_tables, seq_first_row, seq_start_pos, head_bias, status)
    n = q.shape[0]
    assert q.dtype == out.dtype == kcache.dtype == vcache.dtype == torch.bfloat16
    assert q.shape == (n, heads * dim) and out.shape == (n, heads * vdim) and q.is_contiguous() and out.is_contiguous()
    assert block_tables.is_contiguous() and seq_first_row.shape[0] == seq_start_pos.shape[0] + 1
    assert head_bias is None or (head_bias.dtype == torch.float32 and head_bias.numel() == heads)
    _call("gb_sigmoid_attention_tiles", _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), block_tables.shape[1],
          _ptr(seq_first_row), _ptr(seq_start_pos), _ptr(head_bias), seq_start_pos.shape[0], max(int(max_rows_per_seq), 1), heads,
          kv_heads, dim, vdim, page_size, kcache.shape[0], float(scale), int(window) if window else 0, _ptr(status), _stream())


# ------------------------------------------------------- softmax attention with a distance bias, a sink and an output gate
def _sink_args(r1, r2, sink, gate, heads):
    assert (r1 is None) == (r2 is None)
    for t in (r1, r2, sink):
        assert t is None or (t.dtype == torch.float32 and t.numel() == heads)
    assert gate is None or (gate.dtype == torch.float32 and gate.shape[1] == heads and gate.stride(1) == 1)
    return _ptr(r1), _ptr(r2), _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0


def sink_attention_rows(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                        row_seq: torch.Tensor, positions: torch.Tensor, *, r1: Optional[torch.Tensor], r2: Optional[torch.Tensor],
                        sink: Optional[torch.Tensor], gate: Optional[torch.Tensor], heads: int, kv_heads: int, dim: int, vdim: int,
                        page_size: int, scale: float, window: Optional[int], status: torch.Tensor) -> None:
    """out[row, head, :] = sigmoid(gate[row, head]) * sum over the row's visible keys j of w_j v_j, the weights a softmax of
    s_j = q . k_j * scale - r1[head] * ln(1 + r2[head] * distance) whose denominator also holds exp(sink[head]). ``r1``/``r2``,
    ``sink`` (float32 [heads]) and ``gate`` (float32 logits [n, heads], rows may be strided) are each optional. One warp per
    (row, head); any row, both dtypes."""
    _cuda(q, out, kcache, vcache, block_tables, row_seq, positions, r1, r2, sink, gate, status)
    n = q.shape[0]
    assert q.shape == (n, heads * dim) and out.shape == (n, heads * vdim) and q.is_contiguous() and out.is_contiguous()
    assert q.dtype == out.dtype == kcache.dtype == vcache.dtype and block_tables.is_contiguous()
    _call("gb_sink_attention_rows", _ptr(q), _ptr(out), _dt(q), _ptr(kcache), _ptr(vcache), _ptr(block_tables), block_tables.shape[1],
          _ptr(row_seq), _ptr(positions), *_sink_args(r1, r2, sink, gate, heads), n, heads, kv_heads, dim, vdim, page_size,
          kcache.shape[0], float(scale), int(window) if window else 0, _ptr(status), _stream())


def sink_attention_decode_supported(dtype: torch.dtype, vdim: int) -> bool:
    return dtype in _DT and bool(lib().gb_sink_attention_decode_supported(vdim * (4 if dtype == torch.float32 else 2)))


def sink_attention_decode(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                          row_seq: torch.Tensor, positions: torch.Tensor, *, r1: Optional[torch.Tensor], r2: Optional[torch.Tensor],
                          sink: Optional[torch.Tensor], gate: Optional[torch.Tensor], heads: int, kv_heads: int, dim: int, vdim: int,
                          page_size: int, scale: float, window: Optional[int], status: torch.Tensor) -> None:
    """``sink_attention_rows`` for single decoded tokens: a block of eight warps per (row, head) that share the row's keys,
    each with a running maximum of its own, and meet in a fixed order; a value row must be 64, 128, 256 or 512 bytes
    (``sink_attention_decode_supported``)."""
    _cuda(q, out, kcache, vcache, block_tables, row_seq, positions, r1, r2, sink, gate, status)
    n = q.shape[0]
    assert q.shape == (n, heads * dim) and out.shape == (n, heads * vdim) and q.is_contiguous() and out.is_contiguous()
    assert q.dtype == out.dtype == kcache.dtype == vcache.dtype and block_tables.is_contiguous()
    _call("gb_sink_attention_decode", _ptr(q), _ptr(out), _dt(q), _ptr(kcache), _ptr(vcache), _ptr(block_tables),
          block_tables.shape[1], _ptr(row_seq), _ptr(positions), *_sink_args(r1, r2, sink, gate, heads), n, heads, kv_heads, dim, vdim,
          page_size, kcache.shape[0], float(scale), int(window) if window else 0, _ptr(status), _stream())


def sink_attention_tiles_supported(dtype: torch.dtype, dim: int, vdim: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib().gb_sink_attention_tiles_supported(dim, vdim))


def sink_attention_tiles(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                         seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor, max_rows_per_seq: int, *,
                         r1: Optional[torch.Tensor], r2: Optional[torch.Tensor], sink: Optional[torch.Tensor],
                         gate: Optional[torch.Tensor], heads: int, kv_heads: int, dim: int, vdim: int, page_size: int, scale: float,
                         window: Optional[int], status: torch.Tensor) -> None:
    """``sink_attention_rows`` for runs of consecutive rows (prompt portions) in bfloat16 on the tensor cores: a block
    takes 64 rows of one request and one head; ``max_rows_per_seq`` bounds the rows a request brings (it sizes the grid)."""
    _cuda(q, out, kcache, vcache, block_tables, seq_first_row, seq_start_pos, r1, r2, sink, gate, status)
    n = q.shape[0]
    assert q.dtype == out.dtype == kcache.dtype == vcache.dtype == torch.bfloat16
    assert q.shape == (n, heads * dim) and out.shape == (n, heads * vdim) and q.is_contiguous() and out.is_contiguous()
    assert block_tables.is_contiguous() and seq_first_row.shape[0] == seq_start_pos.shape[0] + 1
    _call("gb_sink_attention_tiles", _ptr(q), _ptr(out), _ptr(kcache), _ptr(vcache), _ptr(block_tables), block_tables.shape[1],
          _ptr(seq_first_row), _ptr(seq_start_pos), *_sink_args(r1, r2, sink, gate, heads), seq_start_pos.shape[0],
          max(int(max_rows_per_seq), 1), heads, kv_heads, dim, vdim, page_size, kcache.shape[0], float(scale),
          int(window) if window else 0, _ptr(status), _stream())


# ------------------------------------------------------------------------------------------------ minGRU
def mingru_scan(proj: torch.Tensor, bias_z: torch.Tensor, bias_x: torch.Tensor, state: torch.Tensor, state_off: int, out: torch.Tensor,
                seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor, seq_slots: torch.Tensor, width: int, write_state: bool,
                status: torch.Tensor, max_rows: int = 0) -> None:
    """S_t = (1 - z_t) S_(t-1) + z_t c_t along each request's rows, from and to ``width`` float32 numbers at ``state_off``
    of the request's slot; z = sigmoid(proj[:, :width] + bias_z), c from u = proj[:, width:2 width] + bias_x (u + 1/2 where
    u >= 0, sigmoid(u) elsewhere), out = S_t * silu(proj[:, 2 width:3 width]). proj float32 (a column slice is allowed).
    ``max_rows``: a bound on the rows any request brings in this step (0: unknown, the rows of the step): it sizes the blocks."""
    _cuda(proj, bias_z, bias_x, state, out, seq_first_row, seq_start_pos, seq_slots, status)
    n = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.shape[1] == 3 * width and proj.stride(1) == 1
    assert bias_z.dtype == bias_x.dtype == state.dtype == torch.float32 and bias_z.numel() == width and bias_x.numel() == width
    assert state.dim() == 2 and state.is_contiguous() and out.shape == (n, width) and out.stride(1) == 1
    _call("gb_mingru_scan", _ptr(proj), proj.stride(0), _ptr(bias_z), _ptr(bias_x), _ptr(state), state.stride(0), state_off, _ptr(out),
          out.stride(0), _dt(out), _ptr(seq_first_row), _ptr(seq_start_pos), _ptr(seq_slots), seq_start_pos.shape[0], width,
          state.shape[0], 1 if write_state else 0, int(max_rows) if max_rows > 0 else n, _ptr(status), _stream())


# ------------------------------------------------------------------------------------------- routed experts
def moe_route(h: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], w_gate: Optional[torch.Tensor],
              positions: torch.Tensor, top: int, groups: int, keep: int, route_scale: float, choice: torch.Tensor,
              weight: torch.Tensor, gate: Optional[torch.Tensor], router_bias: Optional[torch.Tensor] = None,
              softmax_chosen: bool = False) -> None:
    """Per row: float32 router logits, sigmoid scores, the ``top`` experts by score + correction among the ``keep`` best of
    ``groups`` runs of neighbouring experts, weights score * route_scale; ``gate`` = sigmoid(w_gate . h) per row. With
    ``softmax_chosen`` the ``top`` largest logits (plus ``router_bias``, float32 [experts]) win and the weights are the
    softmax over the chosen logits alone."""
    _cuda(h, w_router, correction, w_gate, positions, choice, weight, gate, router_bias)
    assert router_bias is None or (softmax_chosen and router_bias.dtype == torch.float32 and router_bias.numel() == w_router.shape[0])
    n, d = h.shape
    E = w_router.shape[0]
    assert h.is_contiguous() and w_router.dtype == torch.float32 and w_router.shape == (E, d) and w_router.is_contiguous()
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == E)
    assert w_gate is None or (w_gate.dtype == torch.float32 and w_gate.numel() == d and gate is not None)
    assert choice.dtype == torch.int32 and choice.shape == (n, top) and choice.is_contiguous()
    assert weight.dtype == torch.float32 and weight.shape == (n, top) and weight.is_contiguous()
    assert gate is None or (gate.dtype == torch.float32 and gate.numel() >= n)
    _call("gb_moe_route", _ptr(h), _dt(h), d, _ptr(w_router), _ptr(correction), _ptr(w_gate), _ptr(positions), n, E, top, groups, keep,
          float(route_scale), _ptr(choice), _ptr(weight), _ptr(gate), _ptr(router_bias), 1 if softmax_chosen else 0, _stream())


def moe_expert_rows(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, experts: int, choice: torch.Tensor,
                    positions: torch.Tensor, pair: torch.Tensor) -> None:
    """pair[row, k, :] = W_down[e] relu(W_up[e] h[row])^2 with e = choice[row, k]; w_up [experts * ff, d] and w_down
    [experts * d, ff] hold the experts' matrices stacked by rows; one block per (row, k)."""
    _cuda(h, w_up, w_down, choice, positions, pair)
    n, d = h.shape
    top = choice.shape[1]
    ff = w_up.shape[0] // experts
    assert h.dtype == w_up.dtype == w_down.dtype and h.is_contiguous() and w_up.is_contiguous() and w_down.is_contiguous()
    assert w_up.shape == (experts * ff, d) and w_down.shape == (experts * d, ff)
    assert pair.dtype == torch.float32 and pair.shape == (n, top * d) and pair.is_contiguous()
    _call("gb_moe_expert_rows", _ptr(h), _dt(h), d, _ptr(w_up), _ptr(w_down), ff, _ptr(choice), _ptr(positions), n, experts, top,
          _ptr(pair), _stream())


def moe_expert_halves(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, experts: int, choice: torch.Tensor,
                       positions: torch.Tensor, act: torch.Tensor, pair: torch.Tensor, unit=None) -> None:
    """``moe_expert_rows`` as two launches of many blocks per (row, choice), for a handful of rows: act float32 [n, top * ff]
    receives relu(W_up[e] h)^2, pair float32 [n, top * d] the experts' outputs. ``unit`` = (limit, slope): the experts are
    clamped gated units, ``w_up`` [experts * 2 ff, d] holds gate row f and up row f of an expert as its rows 2f and 2f + 1,
    and act receives g * sigmoid(slope g) * (u + 1)."""
    _cuda(h, w_up, w_down, choice, positions, act, pair)
    n, d = h.shape
    top = choice.shape[1]
    ff = w_up.shape[0] // experts // (2 if unit else 1)
    assert h.dtype == w_up.dtype == w_down.dtype and h.is_contiguous() and w_up.is_contiguous() and w_down.is_contiguous()
    assert w_up.shape == (experts * ff * (2 if unit else 1), d) and w_down.shape == (experts * d, ff) and choice.is_contiguous()
    assert act.dtype == pair.dtype == torch.float32 and act.shape == (n, top * ff) and pair.shape == (n, top * d)
    assert act.is_contiguous() and pair.is_contiguous()
    _call("gb_moe_expert_halves", _ptr(h), _dt(h), d, _ptr(w_up), _ptr(w_down), ff, _ptr(choice), _ptr(positions), n, experts, top,
          _ptr(act), _ptr(pair), 1 if unit else 0, float(unit[0]) if unit else 0.0, float(unit[1]) if unit else 0.0, _stream())
    global launch_count
    launch_count += 1


def moe_grouped_supported(dtype: torch.dtype, d: int, ff: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib().gb_moe_grouped_supported(d, ff))


def moe_experts_grouped(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, experts: int, choice: torch.Tensor,
                        positions: torch.Tensor, tables: torch.Tensor, act: torch.Tensor, pair: torch.Tensor, unit=None) -> None:
    """The chosen experts of many rows as grouped products on the tensor cores (bfloat16): the (row, choice) pairs are
    sorted by expert (``tables`` int32 [2 * (experts + 1) + n * top] is the sort's scratch), then one launch computes
    act = relu(W_up[e] h)^2 for all pairs (bfloat16 [n, top * ff], in sorted order) and one pair = W_down[e] act
    (float32 [n, top * d], in pair order). ``unit`` as in ``moe_expert_halves``: the up product then has 2 ff outputs per
    expert, and its epilogue forms one unit from every two neighbours."""
    _cuda(h, w_up, w_down, choice, positions, tables, act, pair)
    n, d = h.shape
    top = choice.shape[1]
    up_rows = w_up.shape[0] // experts
    ff = up_rows // (2 if unit else 1)
    P = n * top
    assert h.dtype == w_up.dtype == w_down.dtype == act.dtype == torch.bfloat16 and pair.dtype == torch.float32
    assert h.is_contiguous() and w_up.is_contiguous() and w_down.is_contiguous() and act.is_contiguous() and pair.is_contiguous()
    assert w_up.shape == (experts * up_rows, d) and w_down.shape == (experts * d, ff) and choice.is_contiguous()
    assert act.shape == (n, top * ff) and pair.shape == (n, top * d)
    assert tables.dtype == torch.int32 and tables.is_contiguous() and tables.numel() >= 2 * (experts + 1) + P
    offsets, tile_start, order = tables[:experts + 1], tables[experts + 1:2 * (experts + 1)], tables[2 * (experts + 1):]
    _call("gb_moe_sort", _ptr(choice), _ptr(positions), n, experts, top, _ptr(offsets), _ptr(tile_start), _ptr(order), _stream())
    _call("gb_moe_grouped_gemm", _ptr(h), d, _ptr(w_up), up_rows, d, _ptr(order), _ptr(offsets), _ptr(tile_start), experts, top, P,
          _ptr(act), ff, 1, 1 if unit else 0, float(unit[0]) if unit else 0.0, float(unit[1]) if unit else 0.0, _stream())
    _call("gb_moe_grouped_gemm", _ptr(act), ff, _ptr(w_down), d, ff, _ptr(order), _ptr(offsets), _ptr(tile_start), experts, top, P,
          _ptr(pair), d, 0, 0, 0.0, 0.0, _stream())


def moe_combine(pair: torch.Tensor, weight: torch.Tensor, shared: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                positions: torch.Tensor, out: torch.Tensor, accumulate: bool) -> None:
    """out[row] (+)= sum_k weight[row, k] * pair[row, k] + gate[row] * shared[row]; float32, the sums in a fixed order."""
    _cuda(pair, weight, shared, gate, positions, out)
    n, d = out.shape
    top = weight.shape[1]
    assert pair.dtype == weight.dtype == out.dtype == torch.float32 and pair.shape == (n, top * d) and out.stride(1) == 1
    assert shared is None or (shared.dtype == torch.float32 and shared.shape == (n, d) and shared.stride(1) == 1)
    _call("gb_moe_combine", _ptr(pair), _ptr(weight), top, _ptr(shared), shared.stride(0) if shared is not None else 0, _ptr(gate),
          _ptr(positions), _ptr(out), out.stride(0), n, d, 1 if accumulate else 0, _stream())


# ------------------------------------------------------------------------------ attention whose heads exchange their weights
def bias_rope_write(qkv: torch.Tensor, bias: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor], positions: torch.Tensor,
                    slots: torch.Tensor, q_out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, heads: int, kv_heads: int,
                    dim: int, vdim: int, rot: int, page_size: int, write_kv: bool, status: torch.Tensor) -> None:
    """From the float32 sums of the stacked projection q | k | v: ``bias`` (float32, one number per column, or None) is added,
    the first ``rot`` channels of every query and key head are rotated (channel i with channel i + rot/2, by the (cos, sin) of
    ``cos_sin`` [positions, rot/2, 2] at the row's position), q goes to ``q_out`` [n, heads * dim], k and v into the paged
    cache at each row's slot."""
    _cuda(qkv, bias, cos_sin, positions, slots, q_out, kcache, vcache, status)
    n = qkv.shape[0]
    cols = (heads + kv_heads) * dim + kv_heads * vdim
    assert qkv.dtype == torch.float32 and qkv.stride(1) == 1 and qkv.shape[1] == cols
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == cols and bias.is_contiguous())
    assert q_out.shape == (n, heads * dim) and q_out.is_contiguous() and q_out.dtype == kcache.dtype == vcache.dtype
    assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape[-1] == dim and vcache.shape[-1] == vdim
    assert rot == 0 or (cos_sin is not None and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
                        and tuple(cos_sin.shape[1:]) == (rot // 2, 2))
    _call("gb_bias_rope_write", _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(cos_sin), cos_sin.shape[0] if cos_sin is not None else 0,
          _ptr(positions), _ptr(slots), _ptr(q_out), _ptr(kcache), _ptr(vcache), _dt(q_out), n, heads, kv_heads, dim, vdim, rot, page_size,
          kcache.shape[0] * page_size, 1 if write_kv else 0, _ptr(status), _stream())


def talking_attention_rows(q: torch.Tensor, wide: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                           row_seq: torch.Tensor, positions: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
                           value_heads: int, page_size: int, scale: float, softcap: Optional[float], unit_sink: bool,
                           window: Optional[int], status: torch.Tensor) -> None:
    """wide[row, g, c, :] = sum over the row's visible keys j of w_g(j) * v_c(j), float32 [n, heads * value_heads * vdim], with
    w_g the softmax of head g's (capped) scores whose denominator holds one more unit when ``unit_sink``; ``value_heads`` is
    ``kv_heads`` (every key/value head's values, what a mix of the heads needs) or 1 (the head's own). One warp per (row, head)."""
    _cuda(q, wide, kcache, vcache, block_tables, row_seq, positions, status)
    n = q.shape[0]
    assert q.shape == (n, heads * dim) and q.is_contiguous() and q.dtype == kcache.dtype == vcache.dtype
    assert wide.dtype == torch.float32 and wide.shape == (n, heads * value_heads * vdim) and wide.is_contiguous()
    assert block_tables.is_contiguous() and kcache.is_contiguous() and vcache.is_contiguous()
    _call("gb_talking_attention_rows", _ptr(q), _ptr(wide), _dt(q), _ptr(kcache), _ptr(vcache), _ptr(block_tables), block_tables.shape[1],
          _ptr(row_seq), _ptr(positions), n, heads, kv_heads, dim, vdim, value_heads, page_size, kcache.shape[0], float(scale),
          float(softcap or 0.0), 1.0 if unit_sink else 0.0, int(window or 0), _ptr(status), _stream())


def talking_attention_decode_supported(dtype: torch.dtype, heads: int, kv_heads: int, vdim: int, value_heads: int) -> bool:
    return dtype in _DT and bool(lib().gb_talking_attention_decode_plan(heads, kv_heads, vdim, value_heads))


def talking_decode_shares(n: int, heads: int, kv_heads: int, vdim: int, value_heads: int, reach: int) -> int:
    """Into how many shares the decoding kernel cuts a row's keys: enough blocks for two per multiprocessor, no share shorter
    than 256 keys, at most 16."""
    plan = lib().gb_talking_attention_decode_plan(heads, kv_heads, vdim, value_heads)
    blocks = max(1, n * (heads // max(plan % 10000 // 100, 1)) * max(plan // 10000, 1))
    return int(max(1, min(16, -(-296 // blocks), max(1, reach // 256), 4096 // heads)))


def talking_attention_decode(q: torch.Tensor, wide: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                             row_seq: torch.Tensor, positions: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
                             value_heads: int, page_size: int, scale: float, softcap: Optional[float], unit_sink: bool,
                             window: Optional[int], status: torch.Tensor, shares: int = 1, ml: Optional[torch.Tensor] = None) -> None:
    """``talking_attention_rows`` for steps of single decoded tokens: a block of eight warps per (row, up to eight heads of a
    key/value group, share of the keys) that take the keys in turn and merge in shared memory; a key row is read once for the
    block's heads. With ``shares`` > 1 ``wide`` is float32 [shares * n, heads * value_heads * vdim] (the shares' unnormalised
    sums, share by share) and ``ml`` float32 [shares * n, heads * 2] their maxima and denominators: ``talk_combine`` merges them."""
    _cuda(q, wide, kcache, vcache, block_tables, row_seq, positions, status, ml)
    n = q.shape[0]
    assert q.shape == (n, heads * dim) and q.is_contiguous() and q.dtype == kcache.dtype == vcache.dtype
    assert wide.dtype == torch.float32 and wide.numel() == shares * n * heads * value_heads * vdim and wide.is_contiguous()
    assert shares == 1 or (ml is not None and ml.dtype == torch.float32 and ml.numel() == shares * n * heads * 2 and ml.is_contiguous())
    assert block_tables.is_contiguous() and kcache.is_contiguous() and vcache.is_contiguous() and n <= 2 ** 31 - 1
    _call("gb_talking_attention_decode", _ptr(q), _ptr(wide), _ptr(ml), _dt(q), _ptr(kcache), _ptr(vcache), _ptr(block_tables),
          block_tables.shape[1], _ptr(row_seq), _ptr(positions), n, heads, kv_heads, dim, vdim, value_heads, page_size, kcache.shape[0],
          float(scale), float(softcap or 0.0), 1.0 if unit_sink else 0.0, int(window or 0), int(shares), _ptr(status), _stream())


def talking_attention_tiles_supported(dtype: torch.dtype, dim: int, vdim: int, value_heads: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib().gb_talking_attention_tiles_columns(dim, vdim, value_heads))


def talking_attention_tiles(q: torch.Tensor, wide: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
                            seq_first_row: torch.Tensor, seq_start_pos: torch.Tensor, max_rows_per_seq: int, heads: int, kv_heads: int,
                            dim: int, vdim: int, value_heads: int, page_size: int, scale: float, softcap: Optional[float],
                            unit_sink: bool, window: Optional[int], status: torch.Tensor) -> None:
    """``talking_attention_rows`` for prompt portions in bfloat16 on the tensor cores: 64 rows of one request x one head x up to
    128 columns of the wide value row per block."""
    _cuda(q, wide, kcache, vcache, block_tables, seq_first_row, seq_start_pos, status)
    n = q.shape[0]
    assert q.dtype == kcache.dtype == vcache.dtype == torch.bfloat16 and q.shape == (n, heads * dim) and q.is_contiguous()
    assert wide.dtype == torch.float32 and wide.shape == (n, heads * value_heads * vdim) and wide.is_contiguous()
    assert block_tables.is_contiguous() and kcache.is_contiguous() and vcache.is_contiguous()
    _call("gb_talking_attention_tiles", _ptr(q), _ptr(wide), _ptr(kcache), _ptr(vcache), _ptr(block_tables), block_tables.shape[1],
          _ptr(seq_first_row), _ptr(seq_start_pos), seq_start_pos.shape[0], int(max_rows_per_seq), heads, kv_heads, dim, vdim, value_heads,
          page_size, kcache.shape[0], float(scale), float(softcap or 0.0), 1.0 if unit_sink else 0.0, int(window or 0), _ptr(status),
          _stream())


def talk_combine(wide: torch.Tensor, talk: Optional[torch.Tensor], att: torch.Tensor, positions: torch.Tensor, heads: int, kv_heads: int,
                 vdim: int, value_heads: int, shares: int = 1, ml: Optional[torch.Tensor] = None, unit_sink: bool = True) -> None:
    """att[row, h, :] = sum_g talk[h, g] * wide[row, g, c(h), :] with c(h) the key/value head of h (``talk`` None: head h's own
    result as it is); talk float32 [heads, heads]. With ``shares`` > 1 ``wide`` and ``ml`` are what the decoding kernel left
    share by share, and the shares are merged (with the unit of the denominator, if ``unit_sink``) on the way."""
    _cuda(wide, talk, att, positions, ml)
    n = att.shape[0]
    assert wide.dtype == torch.float32 and wide.numel() == shares * n * heads * value_heads * vdim and wide.is_contiguous()
    assert shares == 1 or (ml is not None and ml.dtype == torch.float32 and ml.numel() == shares * n * heads * 2)
    assert att.shape == (n, heads * vdim) and att.is_contiguous()
    assert talk is None or (talk.dtype == torch.float32 and talk.shape == (heads, heads) and talk.is_contiguous())
    _call("gb_talk_combine", _ptr(wide), _ptr(ml), _ptr(talk), _ptr(att), _dt(att), _ptr(positions), n, heads, kv_heads, vdim, value_heads,
          int(shares), 1.0 if unit_sink else 0.0, _stream())
