"""Python faces of the CUDA kernels: argument checks, then one call into the library.

Every function takes CUDA tensors, launches on torch's current stream and
returns nothing the host has to wait for.  There is no CPU or library
fallback: without a GPU, or without the built library, a call raises.
Sizes a kernel cannot take are refused here with an error that says why.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2
ACTIVATIONS = {"none": ACT_NONE, "gelu_tanh": ACT_GELU_TANH, "gelu_erf": ACT_GELU_ERF}

STATUS_BITS = {
    1: "a token id outside the embedding table",
    2: "a position outside the position table or the sequence limit",
    4: "a block table without a page where the step reads or writes",
    8: "a bounded wait inside a kernel gave up",
}

# Rows up to which a matrix product streams the weights once per group of rows
# instead of tiling: float32 products up to 64 rows (csrc/gemm_simt.cu), then 64x64 tiles in
# IEEE arithmetic on the CUDA cores; bfloat16 products up to 16 rows the weight-streaming mma
# kernel (csrc/gemm_rows_mma.cu), and up to 64 rows too unless the output is wide; otherwise
# tcgen05, clustered (csrc/gemm_tc_rows.cu) or with 128-row tiles (csrc/gemm_tc.cu): bf16_path.
ROWS_STREAMING_LIMIT = 64


class KernelError(RuntimeError):
    pass


_signatures_set = False
_status: dict[int, torch.Tensor] = {}
_launches = 0


def launches() -> int:
    """How many kernels of this library have been launched by this process."""
    return _launches


_loaded = None
_recorder = None  # a LaunchList being filled (see ``recording``)


class LaunchList:
    """The library calls of one step, with their arguments, in order.

    What a step launches depends on its sizes, not on its contents (those lie in device
    buffers whose addresses stay): a step of sizes seen before can issue the recorded calls
    again instead of walking through the parts and the checked wrappers a second time.
    """

    def __init__(self) -> None:
        self.calls: list[tuple] = []  # (library function, arguments without the stream)
        self.launches = 0             # kernels these calls launch
        self.result = None            # whatever the recorded code returned (set by the caller)

    def replay(self) -> None:
        global _launches
        stream = _stream()
        for fn, args in self.calls:
            rc = fn(*args, stream)
            if rc != 0:
                raise KernelError(f"{fn.__name__}: code {rc} when a recorded launch was issued again")
        _launches += self.launches


class _RecordingLib:
    """Stands for the library while a ``LaunchList`` is filled: every launch is made and noted."""

    def __init__(self, lib, into: LaunchList) -> None:
        self._lib, self._into = lib, into

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if name in _QUERIES:
            return fn

        def call(*args):
            self._into.calls.append((fn, args[:-1]))  # the stream is every launch's last argument
            return fn(*args)

        return call


_QUERIES = ("rl_gemm_tc_rows_fits", "rl_gemm_rows_smem_fits", "rl_mlp_fused_slice", "rl_attn_block_fused_fits", "rl_attn_block_fused_cluster",
            "rl_host_memory_on_device", "rl_latent_attention_fits", "rl_latent_decode_fits",
            "rl_moe_max_tiles", "rl_bias_attention_shape", "rl_recurrence_record")  # library functions that launch nothing


class recording:
    """``with recording() as launches:`` notes every library launch made inside."""

    def __enter__(self) -> LaunchList:
        global _recorder
        if _recorder is not None:
            raise KernelError("launches are being recorded already")
        self._list = LaunchList()
        self._before = _launches
        _recorder = _RecordingLib(_lib(), self._list)
        return self._list

    def __exit__(self, *exc) -> None:
        global _recorder
        _recorder = None
        self._list.launches = _launches - self._before


def _lib() -> ctypes.CDLL:
    global _signatures_set, _loaded
    if _recorder is not None:
        return _recorder
    if _loaded is not None:
        return _loaded
    lib = build.load()
    if not _signatures_set:
        P, I, L, F = c_void_p, c_int, c_long, c_float
        lib.rl_embed.argtypes = [I, P, P, P, P, P, I, I, I, I, P, P, I, F, P]
        lib.rl_layernorm.argtypes = [I, P, P, P, P, P, I, I, F, P]
        lib.rl_gemm_simt.argtypes = [I, I, P, L, P, P, P, L, I, I, I, I, I, I, P, P, I, P, P, P,
                                     I, I, I, I, I, I, P, P]
        lib.rl_gemm_rows_bf16.argtypes = [I, P, L, P, P, P, L, I, I, I, I, I, P, L, P, P, F, P, P, I, P, P, P,
                                          I, I, I, I, I, I, P, P]
        lib.rl_gemm_rows_bf16_sample.argtypes = [P, L, P, P, I, I, I, P, L, P, P, F, P, P, P, P, P, P, P, I, P, P, P]
        lib.rl_host_memory_on_device.argtypes = [P]
        lib.rl_host_memory_on_device.restype = ctypes.c_ulonglong
        lib.rl_gemm_rows_bulk_enable.argtypes = [I]
        lib.rl_gemm_rows_bulk_enable.restype = None
        lib.rl_gemm_tc.argtypes = [I, P, L, P, P, P, L, I, I, I, I, I, P, P, I, P, P, P, I, I, I, I, I, I, P, P]
        lib.rl_gemm_tc_sample.argtypes = [P, L, P, P, I, I, I, P, P, P, P, P, P, P, I, P, P, P]
        lib.rl_gemm_tc_cut.argtypes = [I, P, L, P, P, P, L, I, I, I, I, I, P, P, I, P, P, P, I, I, I, I, I, I, P, I, I, P]
        lib.rl_gemm_tc_rows.argtypes = [I, P, L, P, P, P, L, I, I, I, I, I, P, P, I, P, P, P, I, I, I, I, I, I, P, P]
        lib.rl_gemm_tc_rows_fits.argtypes = [I, I, I]
        lib.rl_gemm_rows_smem.argtypes = [I, P, L, P, P, P, L, I, I, I, I, I, P, P, I, P, P, P, I, I, I, I, I, I, P, P]
        lib.rl_gemm_rows_smem_fits.argtypes = [I, I, I, I, I, I, I]
        lib.rl_copy_to_device.argtypes = [P, P, L, P]
        lib.rl_event_record.argtypes = [P, P]
        lib.rl_attention.argtypes = [I, P, L, P, P, I, P, P, P, P, L, I, I, I, I, I, F, P, I, P, I, P, I, I, I, P, P, I, L, I, I, P, P]
        lib.rl_kv_write.argtypes = [I, P, P, L, P, P, I, P, P, P, I, I, I, I, I, P, P]
        lib.rl_sample.argtypes = [P, L, I, I, P, P, P, P, P, P, P, I, P, P, I, P]
        lib.rl_mlp_fused_slice.argtypes = [I, I, I, I]
        lib.rl_attn_block_fused_fits.argtypes = [I, I, I, I]
        lib.rl_attn_block_fused_cluster.argtypes = [I, I, I]
        lib.rl_attn_block_fused.argtypes = [P, L, P, P, F, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, P, P]
        lib.rl_mlp_fused.argtypes = [P, L, P, L, P, P, F, P, P, P, P, I, I, I, I, I, P, P]
        lib.rl_rmsnorm.argtypes = [I, P, L, P, P, P, L, I, I, F, P]
        lib.rl_rmsnorm_add.argtypes = [P, L, P, P, L, P, L, I, I, F, F, P]
        lib.rl_cast_rows.argtypes = [P, P, L, P]
        lib.rl_latent_attention_fits.argtypes = [I, I, I]
        lib.rl_latent_decode_fits.argtypes = [I, I, I]
        lib.rl_latent_kv_write.argtypes = [I, P, L, P, F, P, I, P, P, I, P, P, P, I, I, I, I, I, I, F, P, P]
        lib.rl_latent_q_rope.argtypes = [I, P, L, I, I, P, L, I, I, I, I, P, P, I, I, F, P]
        lib.rl_latent_attention.argtypes = [I, P, L, P, P, I, P, P, P, P, L, P, I, I, I, I, F, P, I, P, I, I, I, P, P, I, P, P]
        lib.rl_head_linear.argtypes = [I, P, L, L, P, L, L, L, P, L, L, I, I, I, I, P, L, L, P]
        lib.rl_gated_act.argtypes = [I, P, L, I, P, L, I, I, I, F, F, P]
        lib.rl_token_gate.argtypes = [I, P, L, P, P, L, I, I, P, L, I, I, I, P, I, P, P]
        lib.rl_moe_select.argtypes = [P, L, P, I, I, I, I, I, I, P, P, P, P]
        lib.rl_moe_plan.argtypes = [P, P, P, P, P, P, P, P, P, P, I, I, I, P]
        lib.rl_moe_max_tiles.argtypes = [I, I]
        lib.rl_moe_experts.argtypes = [I, P, L, P, P, P, P, P, P, P, P, P, L, P, P, L, I, I, I, I, I, I, F, F, I, P]
        lib.rl_embed_pair.argtypes = [I, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P, P, P, I, P]
        lib.rl_rmsnorm_add_norm.argtypes = [I, P, L, P, P, L, P, P, L, I, I, F, F, P]
        lib.rl_recurrence.argtypes = [I, I, P, L, I, I, I, I, I, I, P, P, P, I, P, P, P, L, P, P, P, P, I, I, I, I, I, F, F, F,
                                      L, I, F, F, F, F, P, P]
        lib.rl_recurrence_record.argtypes = [I, I, I, P, P, P]
        lib.rl_bias_attention_shape.argtypes = [I, I, P, P]
        lib.rl_bias_attention.argtypes = [I, I, P, L, P, L, P, P, L, P, P, P, P, I, I, P, I, P, L, I, I, I, I, I, I, I, I,
                                          F, F, I, P, P, I, P, P, I, I, P, P, I, P]
        lib.rl_qkv_norm_rotate.argtypes = [P, L, P, L, P, L, P, P, P, P, I, I, I, I, I, I, I, I, F,
                                           I, P, P, L, P, P, I, I, I, I, P, P]
        lib.rl_stream_inject.argtypes = [P, L, P, P, L, P, L, I, I, P]
        lib.rl_gate_mul.argtypes = [I, P, L, P, L, I, I, P]
        lib.rl_stream_inject_norm.argtypes = [I, P, L, P, P, L, P, L, P, F, P, L, I, I, P]
        lib.rl_moe_table_select.argtypes = [P, P, I, I, I, I, F, P, P, P, P, I, P, P]
        lib.rl_moe_table_route.argtypes = [P, P, I, I, I, I, F, P, P, P, P, P, P, P, P, I, P, P]
        lib.rl_gated_join_norm.argtypes = [P, L, F, P, L, F, P, L, P, P, P, L, P, L, I, I, F, F, P]
        lib.rl_bias_kv_store.argtypes = [I, P, L, P, L, P, P, I, P, P, L, P, P, P, I, I, I, I, I, I, I, I, P, P]
        for name in ("rl_rmsnorm", "rl_rmsnorm_add", "rl_cast_rows", "rl_latent_attention_fits", "rl_latent_decode_fits",
                     "rl_latent_kv_write", "rl_latent_q_rope", "rl_latent_attention", "rl_head_linear", "rl_gated_act",
                     "rl_token_gate", "rl_moe_select", "rl_moe_plan", "rl_moe_max_tiles", "rl_moe_experts", "rl_embed_pair",
                     "rl_rmsnorm_add_norm", "rl_recurrence", "rl_recurrence_record", "rl_bias_attention_shape", "rl_bias_attention",
                     "rl_bias_kv_store", "rl_qkv_norm_rotate", "rl_gated_join_norm", "rl_stream_inject", "rl_gate_mul",
                     "rl_moe_table_select", "rl_stream_inject_norm", "rl_moe_table_route"):
            getattr(lib, name).restype = I
        for name in ("rl_copy_to_device", "rl_event_record", "rl_embed", "rl_layernorm", "rl_gemm_simt", "rl_gemm_tc", "rl_gemm_tc_sample", "rl_gemm_tc_cut", "rl_gemm_tc_rows", "rl_gemm_tc_rows_fits",
                     "rl_gemm_rows_smem", "rl_gemm_rows_smem_fits",
                     "rl_gemm_rows_bf16", "rl_gemm_rows_bf16_sample", "rl_attention", "rl_kv_write", "rl_sample", "rl_mlp_fused_slice", "rl_mlp_fused",
                     "rl_attn_block_fused_fits", "rl_attn_block_fused_cluster", "rl_attn_block_fused"):
            getattr(lib, name).restype = I
        _signatures_set = True
    _loaded = lib
    return lib


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {t.dtype}; float32 or bfloat16")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (asked for at every launch: the raw call costs a
    tenth of a microsecond, ``torch.cuda.current_stream()`` several)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, name: str, dtype: torch.dtype | None = None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _ok(rc: int, what: str) -> None:
    global _launches
    _launches += 1
    if rc != 0:
        if rc > 0:
            raise KernelError(f"{what}: CUDA error {rc} at launch")
        raise KernelError(f"{what}: refused its arguments (code {rc})")


def status_word(device: torch.device) -> torch.Tensor:
    """The int32 word kernels OR error bits into (one per device)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device: torch.device) -> None:
    """Read the status word (waits for the stream) and raise if a kernel flagged its inputs."""
    word = status_word(device)
    bits = int(word.item())
    if bits:
        word.zero_()
        why = "; ".join(text for bit, text in STATUS_BITS.items() if bits & bit)
        raise KernelError(f"a kernel refused part of its input: {why}")


def copy_to_device(dst: torch.Tensor, src: torch.Tensor, n: int, offset: int = 0) -> None:
    """dst[offset:offset + n] = src[offset:offset + n] for a device tensor and a pinned host tensor
    of the same element type (both contiguous), ordered on the current stream; the host side must
    stay as it is until the stream has passed the copy."""
    if not dst.is_cuda or src.is_cuda or not src.is_pinned() or dst.dtype != src.dtype:
        raise KernelError("copy_to_device: a device tensor and a pinned host tensor of one element type are needed")
    if offset < 0 or n < 0 or offset + n > min(dst.numel(), src.numel()):
        raise KernelError("copy_to_device: the range lies outside the tensors")
    size = dst.element_size()
    rc = _lib().rl_copy_to_device(dst.data_ptr() + offset * size, src.data_ptr() + offset * size, n * size, _stream())
    if rc != 0:  # not a kernel: it does not count as a launch
        raise KernelError(f"copy_to_device: CUDA error {rc}")


def copy_to_device_raw(dst_ptr: int, src_ptr: int, n_bytes: int) -> None:
    """The same for addresses the caller has checked once (buffers it keeps for the purpose):
    nothing is looked up or checked here, a step makes two such copies."""
    rc = _lib().rl_copy_to_device(dst_ptr, src_ptr, n_bytes, _stream())
    if rc != 0:
        raise KernelError(f"copy_to_device: CUDA error {rc}")


def record_event(event: "torch.cuda.Event") -> None:
    """``event.record()`` on the current stream; after the event's first use, by the plain runtime
    call on its handle (the framework's own call looks the stream object up each time)."""
    handle = event.cuda_event
    if not handle:
        event.record()
        return
    rc = _lib().rl_event_record(handle, _stream())
    if rc != 0:
        raise KernelError(f"record_event: CUDA error {rc}")


def embed(token_ids, positions, table, pos_table, out, feedback=None, scale: float = 1.0) -> None:
    """out[n] = scale * table[token_ids[n]] (+ pos_table[positions[n]]), float32 [tokens, hidden].
    With ``feedback`` (int32), an id -(r+1) is replaced on the device by ``feedback[r]``."""
    _need(token_ids, "token_ids", torch.int32)
    _need(table, "table")
    _need(out, "out", torch.float32)
    n, hidden = out.shape
    if table.shape[1] != hidden:
        raise KernelError("table width differs from out")
    n_pos = 0
    if pos_table is not None:
        _need(pos_table, "pos_table", table.dtype)
        _need(positions, "positions", torch.int32)
        n_pos = pos_table.shape[0]
    rc = _lib().rl_embed(_code(table), _ptr(token_ids), _ptr(positions), _ptr(table), _ptr(pos_table),
                         _ptr(out), n, hidden, table.shape[0], n_pos, _ptr(status_word(out.device)),
                         _ptr(feedback), 0 if feedback is None else feedback.numel(), float(scale), _stream())
    _ok(rc, "embed")


def layernorm(x, gamma, beta, eps: float, out, rows=None) -> None:
    """out[i] = LayerNorm(x[rows[i]] or x[i]) * gamma + beta; x float32, out float32 or bfloat16."""
    _need(x, "x", torch.float32)
    _need(gamma, "gamma", torch.float32)
    if beta is not None:
        _need(beta, "beta", torch.float32)
    _need(out, "out")
    hidden = x.shape[1]
    n_out = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() < n_out:
            raise KernelError("rows shorter than out")
    elif x.shape[0] < n_out:
        raise KernelError("x has fewer rows than out")
    if out.shape[1] != hidden or gamma.numel() != hidden:
        raise KernelError("layernorm: widths differ")
    rc = _lib().rl_layernorm(_code(out), _ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out),
                             n_out, hidden, float(eps), _stream())
    if rc == -2:
        raise KernelError(f"layernorm: a row of {hidden} floats does not fit in shared memory")
    _ok(rc, "layernorm")


_device_facts: dict[int, tuple[int, int]] = {}
device_facts_given: tuple[int, int] | None = None  # set by tests that plan for a device they do not have


def device_facts(device: torch.device | None = None) -> tuple[int, int]:
    """(SMs, bytes of shared memory an SM has) of the device the kernels run on, asked once."""
    if device_facts_given is not None:
        return device_facts_given
    key = torch.cuda.current_device() if device is None or device.index is None else device.index
    have = _device_facts.get(key)
    if have is None:
        props = torch.cuda.get_device_properties(key)
        have = _device_facts[key] = (int(props.multi_processor_count), int(props.shared_memory_per_multiprocessor))
    return have


def sm_count(device: torch.device | None = None) -> int:
    return device_facts(device)[0]


def bf16_path(rows: int, n_out: int, k: int, *, residual: bool = False, out_f32: bool = False, act: int = ACT_NONE,
              to_cache: bool = False) -> str:
    """Which kernel a bfloat16 product of these sizes runs on (measured on B200 at the widths of
    GPT-2): up to 16 rows the weight-streaming mma kernel; 17 to 64 rows the kernel that keeps
    both operands in shared memory, unless the output alone has tiles enough to fill the SMs (the
    head: tcgen05 tiles) or its sizes do not fit (then the weight-streaming kernel, or for a long
    inner size the clustered tcgen05 kernel); up to 128 rows the clustered kernel when the output
    is too narrow to give the tiled kernel work; beyond, tcgen05 tiles."""
    if rows < 17:
        return "mma"
    if rows <= 64:
        if -(-n_out // 64) >= sm_count():
            return "tc"
        if ROWS_IN_SHARED_MEMORY and _lib().rl_gemm_rows_smem_fits(rows, n_out, k, int(residual), int(out_f32), act,
                                                                   int(to_cache)):
            return "smem"
        if rows > 32 and k >= 2048 and _lib().rl_gemm_tc_rows_fits(rows, n_out, k):
            return "tcr"
        return "mma"
    if rows <= 128 and n_out <= 1024 and _lib().rl_gemm_tc_rows_fits(rows, n_out, k):
        return "tcr"
    return "tc"


# The kernel of 17 to 64 rows that stages both operands in shared memory (csrc/gemm_rows_smem.cu);
# switched off, those products run as they did without it (for comparisons).
ROWS_IN_SHARED_MEMORY = True


def product_writes_cache(rows: int, dtype: torch.dtype, n_out: int = 0, k: int = 0) -> bool:
    """Whether ``linear`` on this many rows (``n_out`` output columns, inner size ``k``) runs a
    kernel into which the cache write after it can be fused."""
    if dtype == torch.float32:
        return rows <= ROWS_STREAMING_LIMIT
    return True  # every bfloat16 product kernel can scatter keys and values


# Most rows, and longest rows, for which a LayerNorm is computed inside the product that
# consumes it (csrc/gemm_rows_mma.cu).
FUSED_NORM_MAX_ROWS = 16
FUSED_NORM_MAX_WIDTH = 1024


class NormInput:
    """The input of a bfloat16 product given as "LayerNorm of these float32 rows": the row
    kernel normalises them itself (``linear(NormInput(...), ...)``)."""

    def __init__(self, x, gamma, beta, eps: float) -> None:
        self.x, self.gamma, self.beta, self.eps = x, gamma, beta, float(eps)

    @staticmethod
    def possible(rows: int, width: int, dtype: torch.dtype) -> bool:
        return dtype == torch.bfloat16 and rows <= FUSED_NORM_MAX_ROWS and width <= FUSED_NORM_MAX_WIDTH and width % 4 == 0


class KvTarget:
    """Where the key and value columns of a packed qkv product go instead of the output buffer."""

    def __init__(self, pool, block_table, positions, req_of_token, slots, q_width: int, max_pos: int) -> None:
        self.pool, self.block_table = pool, block_table
        self.positions, self.req_of_token, self.slots = positions, req_of_token, slots
        self.q_width, self.max_pos = q_width, max_pos


def linear(a, weight, bias, out, *, act: int = ACT_NONE, residual: bool = False, path: str | None = None,
           kv: KvTarget | None = None, tile_width: int = 0, splits: int = 0) -> None:
    """out = act(a @ weight.T + bias), or out += ... when residual (out float32).

    ``a`` may be a ``NormInput``: the product then normalises float32 rows itself (bfloat16,
    at most 16 rows).  Otherwise
    a [rows, k] (row stride a multiple of 8), weight [n, k] contiguous, both float32 or both
    bfloat16; out [rows, n] of a's dtype or float32.  Which kernel runs: float32 up to 64 rows
    the row kernel, above it 64x64 tiles (both IEEE FFMA); bfloat16 up to 16 rows the
    weight-streaming mma kernel (for a very wide float32 output, a head, its form that is fed by
    bulk copies: the library chooses), above it as ``bf16_path`` says.  ``path`` (for tests) forces
    ``"rows"``, ``"tile"``, ``"mma"``, ``"smem"``, ``"tc"`` or ``"tcr"``.  ``kv``: output columns from
    ``kv.q_width`` on are written into cache pages, not ``out`` (not with ``"tile"``).
    ``tile_width`` and ``splits`` (for tests and measurements, ``"tc"`` only): the columns of an
    output tile, a multiple of 32 up to 256, and the parts the inner size is cut into (1, 2, 3, 4, 6
    or 8: the blocks of a cluster take one each), instead of what the kernel would choose.
    """
    norm = a if isinstance(a, NormInput) else None
    _need(weight, "weight")
    _need(out, "out", contiguous=False)
    if norm is not None:
        _need(norm.x, "norm.x", torch.float32, contiguous=False)
        _need(norm.gamma, "norm.gamma", torch.float32)
        m, k = norm.x.shape
        if weight.dtype != torch.bfloat16 or not NormInput.possible(m, k, torch.bfloat16) or norm.x.stride(1) != 1 \
                or norm.x.stride(0) % 4 or norm.gamma.numel() != k or path not in (None, "mma"):
            raise KernelError("linear: a LayerNorm is fused only into bfloat16 row products of at most "
                              f"{FUSED_NORM_MAX_ROWS} rows of at most {FUSED_NORM_MAX_WIDTH} elements")
        a_dtype, a_ptr, lda = torch.bfloat16, None, 0
        path = "mma"
    else:
        _need(a, "a", weight.dtype, contiguous=False)
        m, k = a.shape
        if a.stride(1) != 1:
            raise KernelError("linear: rows of a must be contiguous")
        if a.stride(0) % 8 != 0 or a.data_ptr() % 16:
            raise KernelError(f"linear: the row stride {a.stride(0)} must be a multiple of 8 and a start on a 16-byte boundary")
        a_dtype, a_ptr, lda = a.dtype, a.data_ptr(), a.stride(0)
    n = weight.shape[0]
    if weight.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise KernelError(f"linear: shapes do not fit: input [{m}, {k}], weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if out.stride(1) != 1:
        raise KernelError("linear: rows of out must be contiguous")
    if k % 8 != 0:
        raise KernelError(f"linear: the inner size {k} must be a multiple of 8")
    if weight.data_ptr() % 16:
        raise KernelError("linear: operands must start on 16-byte boundaries")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != n:
            raise KernelError("linear: bias length differs from the output width")
    if residual and out.dtype != torch.float32:
        raise KernelError("linear: the residual stream is float32")
    if a_dtype == torch.float32 and out.dtype != torch.float32:
        raise KernelError("linear: float32 inputs give float32 outputs")
    bf16 = a_dtype == torch.bfloat16
    if path is None:
        if bf16:
            path = bf16_path(m, n, k, residual=residual, out_f32=out.dtype == torch.float32, act=act, to_cache=kv is not None)
        else:
            path = "rows" if m <= ROWS_STREAMING_LIMIT else "tile"
    if path in ("mma", "tc", "tcr", "smem") and not bf16:
        raise KernelError("linear: the tensor-core kernels take bfloat16 inputs")
    if path == "mma" and m > 64:
        raise KernelError("linear: the mma row kernel takes at most 64 rows")
    if path == "tcr" and not _lib().rl_gemm_tc_rows_fits(m, n, k):
        raise KernelError("linear: the clustered tcgen05 kernel takes at most 128 rows and an inner size that "
                          "fits the shared memory of eight blocks")
    if kv is not None and path == "tile":
        raise KernelError("linear: the 32-bit tile kernel does not write into the cache")
    if kv is not None and (act != ACT_NONE or residual):
        raise KernelError("linear: a product that writes keys and values has no activation and no residual")
    status = _ptr(status_word(out.device))
    kx = (None, None, 0, None, None, None, 0, 0, 0, 0, 0, 0)
    if kv is not None:
        _need(kv.pool, "kv.pool", a_dtype)
        _, two, n_kv, page_size, dh = kv.pool.shape
        if kv.q_width + 2 * n_kv * dh != n:
            raise KernelError("linear: the packed qkv width does not fit the cache's heads")
        kx = (kv.pool.data_ptr(), kv.block_table.data_ptr(), kv.block_table.stride(0), kv.positions.data_ptr(),
              kv.req_of_token.data_ptr(), kv.slots.data_ptr(), kv.q_width, n_kv * dh, dh, page_size, n_kv, kv.max_pos)
    if path == "smem":
        rc = _lib().rl_gemm_rows_smem(_code(out), a_ptr, lda, _ptr(weight), _ptr(bias), _ptr(out),
                                      out.stride(0), m, n, k, act, int(residual), *kx, status, _stream())
        if rc == -2:
            raise KernelError("linear: the shared-memory row kernel takes at most 64 rows, an even output width, and an "
                              "inner size of at most 1024 (longer only for out += ... into float32)")
        _ok(rc, "linear (rows in shared memory)")
    elif path == "tc":
        rc = _lib().rl_gemm_tc_cut(_code(out), a_ptr, lda, _ptr(weight), _ptr(bias), _ptr(out),
                                   out.stride(0), m, n, k, act, int(residual), *kx, status, tile_width, splits, _stream())
        if rc in (-10, -11):
            raise KernelError("linear: the driver refused to encode a TMA tensor map for these operands")
        _ok(rc, "linear (tcgen05)")
    elif path == "tcr":
        rc = _lib().rl_gemm_tc_rows(_code(out), a_ptr, lda, _ptr(weight), _ptr(bias), _ptr(out),
                                    out.stride(0), m, n, k, act, int(residual), *kx, status, _stream())
        if rc in (-10, -11):
            raise KernelError("linear: the driver refused to encode a TMA tensor map for these operands")
        _ok(rc, "linear (tcgen05 rows)")
    elif path == "mma":
        nx = (None, 0, None, None, 0.0)
        if norm is not None:
            nx = (norm.x.data_ptr(), norm.x.stride(0), norm.gamma.data_ptr(), _ptr(norm.beta), norm.eps)
        rc = _lib().rl_gemm_rows_bf16(_code(out), a_ptr, lda, _ptr(weight), _ptr(bias), _ptr(out),
                                      out.stride(0), m, n, k, act, int(residual), *nx, *kx, status, _stream())
        if rc == -6:
            raise KernelError("linear: the rows to normalise must be 16-byte aligned float32")
        _ok(rc, "linear (mma rows)")
    else:
        rows_limit = (1 << 30) if path == "rows" else 0
        rc = _lib().rl_gemm_simt(_code(weight), _code(out), a_ptr, lda, _ptr(weight), _ptr(bias), _ptr(out),
                                 out.stride(0), m, n, k, act, int(residual), rows_limit, *kx, status, _stream())
        _ok(rc, "linear")


class SampleInto:
    """Where a step's next tokens go when the head's product chooses them itself, and the rows'
    sampling options: device tensors whose addresses stay (captured graphs hold them).
    ``out_ids`` int32; ``temperature`` float32 (<= 0: arg-max), ``seeds`` int64, ``counters``
    int32, one entry a row, or all three ``None`` when every row takes the arg-max.
    ``host_ring`` (optional): pinned int32 host memory of ``SAMPLE_RING`` slots of ``ring_stride``
    ids that the kernel writes the ids to as well, with ``ring_step`` (device, one uint32-sized
    int32) counting the launches that have: launch number n (from 0) fills slot
    ``n % SAMPLE_RING``, so that the host needs no copy of its own to see the tokens."""

    def __init__(self, out_ids, temperature=None, seeds=None, counters=None, host_ring=None, ring_step=None) -> None:
        self.out_ids, self.temperature, self.seeds, self.counters = out_ids, temperature, seeds, counters
        self.host_ring, self.ring_step = host_ring, ring_step
        self.ring_address, self.ring_stride = 0, 0
        if host_ring is not None:
            if ring_step is None or not host_ring.is_pinned() or host_ring.dtype != torch.int32 \
                    or host_ring.numel() % SAMPLE_RING or not host_ring.is_contiguous():
                raise KernelError("SampleInto: the host ring is pinned int32 memory of SAMPLE_RING equal slots, "
                                  "with a device counter beside it")
            _need(ring_step, "ring_step", torch.int32)
            self.ring_address = host_memory_on_device(host_ring)
            self.ring_stride = host_ring.numel() // SAMPLE_RING
            if not self.ring_address:
                raise KernelError("SampleInto: the device cannot write to this host memory")


SAMPLE_RING = 4  # slots of a SampleInto's host ring (csrc/gemm_epilogue.cuh)


def host_memory_on_device(t: torch.Tensor) -> int:
    """The address under which kernels reach the pinned host tensor ``t`` (0: they cannot)."""
    if t.is_cuda or not t.is_pinned():
        return 0
    return int(_lib().rl_host_memory_on_device(t.data_ptr()))


# A head's product chooses the tokens in its epilogue where it runs on the weight-streaming
# kernel (up to 16 rows) or on tcgen05 tiles (more rows and an output wide enough to fill the
# SMs: ``bf16_path``); the kernels between them have no such epilogue.
SAMPLING_PRODUCT_MAX_ROWS = 1024  # words of scratch
_sampling_product_bufs: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


def sampling_product_possible(rows: int, n_out: int, k: int, dtype: torch.dtype, with_temperature: bool = False) -> bool:
    """Whether ``linear_sample`` takes these sizes, and is the faster way: on tcgen05 tiles the
    few epilogue threads of a block are slower at the noise of rows with a temperature than the
    sampling kernel after an ordinary product (64 x 50257: 64 against 46 us; the arg-max alone:
    24 against 33), so such batches are left to that."""
    if dtype != torch.bfloat16 or not 0 < rows <= SAMPLING_PRODUCT_MAX_ROWS or k % 8:
        return False
    path = bf16_path(rows, n_out, k, out_f32=True)
    return path == "mma" or (path == "tc" and not with_temperature)


def linear_sample(a, weight, bias, into: SampleInto) -> None:
    """``into.out_ids[r]`` = the token ``sample`` would choose from row r of ``a @ weight.T + bias``
    (arg-max, or with a temperature the arg-max of logit / temperature + Gumbel noise), without
    the logits being written anywhere.  bfloat16, where ``sampling_product_possible``;
    ``a`` may be a ``NormInput`` as for ``linear``.  Rows with top-k or top-p need their logits:
    they are not for this call."""
    norm = a if isinstance(a, NormInput) else None
    _need(weight, "weight", torch.bfloat16)
    n, k = weight.shape
    if norm is not None:
        _need(norm.x, "norm.x", torch.float32, contiguous=False)
        _need(norm.gamma, "norm.gamma", torch.float32)
        m = norm.x.shape[0]
        if not NormInput.possible(m, k, torch.bfloat16) or norm.x.shape[1] != k or norm.x.stride(1) != 1 \
                or norm.x.stride(0) % 4 or norm.gamma.numel() != k:
            raise KernelError("linear_sample: a LayerNorm is fused only into bfloat16 row products of at most "
                              f"{FUSED_NORM_MAX_ROWS} rows of at most {FUSED_NORM_MAX_WIDTH} elements")
        a_ptr, lda = None, 0
        nx = (norm.x.data_ptr(), norm.x.stride(0), norm.gamma.data_ptr(), _ptr(norm.beta), norm.eps)
    else:
        _need(a, "a", torch.bfloat16, contiguous=False)
        m = a.shape[0]
        if a.shape[1] != k or a.stride(1) != 1 or a.stride(0) % 8 or a.data_ptr() % 16:
            raise KernelError("linear_sample: a must be [rows, k] with contiguous rows, a row stride that is a "
                              "multiple of 8 and a start on a 16-byte boundary")
        a_ptr, lda = a.data_ptr(), a.stride(0)
        nx = (None, 0, None, None, 0.0)
    if not sampling_product_possible(m, n, k, torch.bfloat16) or weight.data_ptr() % 16:
        raise KernelError("linear_sample: rows and an output width that the weight-streaming or the tcgen05 product "
                          "takes, an inner size that is a multiple of 8 and weights on a 16-byte boundary")
    path = bf16_path(m, n, k, out_f32=True)
    if norm is not None and path != "mma":
        raise KernelError("linear_sample: a LayerNorm is fused only into the weight-streaming product")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != n:
            raise KernelError("linear_sample: bias length differs from the output width")
    _need(into.out_ids, "out_ids", torch.int32)
    if into.out_ids.numel() < m:
        raise KernelError("linear_sample: out_ids is shorter than the number of rows")
    given = [t is not None for t in (into.temperature, into.seeds, into.counters)]
    if any(given) and not all(given):
        raise KernelError("linear_sample: temperature, seeds and counters come together")
    for t, name, dt in ((into.temperature, "temperature", torch.float32), (into.seeds, "seeds", torch.int64),
                        (into.counters, "counters", torch.int32)):
        if t is not None:
            _need(t, name, dt)
            if t.numel() < m:
                raise KernelError(f"linear_sample: {name} is shorter than the number of rows")
    key = weight.device.index if weight.device.index is not None else torch.cuda.current_device()
    bufs = _sampling_product_bufs.get(key)
    if bufs is None:  # best words and ticket: zero between launches
        bufs = _sampling_product_bufs[key] = (
            torch.zeros(SAMPLING_PRODUCT_MAX_ROWS, dtype=torch.int64, device=weight.device),
            torch.zeros(1, dtype=torch.int32, device=weight.device))
    if into.ring_address and into.ring_stride < m:
        raise KernelError("linear_sample: the host ring's slots are shorter than the number of rows")
    ring = (into.ring_address or None, into.ring_stride, _ptr(into.ring_step) if into.ring_address else None)
    if path == "tc":
        rc = _lib().rl_gemm_tc_sample(a_ptr, lda, _ptr(weight), _ptr(bias), m, n, k, _ptr(into.temperature),
                                      _ptr(into.seeds), _ptr(into.counters), _ptr(into.out_ids), _ptr(bufs[0]),
                                      _ptr(bufs[1]), *ring, _ptr(status_word(weight.device)), _stream())
        if rc in (-10, -11):
            raise KernelError("linear_sample: the driver refused to encode a TMA tensor map for these operands")
        _ok(rc, "linear_sample (tcgen05)")
        return
    rc = _lib().rl_gemm_rows_bf16_sample(a_ptr, lda, _ptr(weight), _ptr(bias), m, n, k, *nx, _ptr(into.temperature),
                                         _ptr(into.seeds), _ptr(into.counters), _ptr(into.out_ids), _ptr(bufs[0]),
                                         _ptr(bufs[1]), *ring, _ptr(status_word(weight.device)), _stream())
    _ok(rc, "linear_sample")


def rows_bulk_kernel(on: bool) -> None:
    """Heads of few rows on the kernel that has their weights copied into shared memory by the
    copy engine (the default), or on the weight-streaming kernel as every other product of few
    rows (for comparisons and measurements)."""
    build.load().rl_gemm_rows_bulk_enable(int(on))


# The fused kernels of a decode layer (csrc/mlp_fused.cu) are taken where their sizes fit;
# switched off, every layer runs as separate products (for comparisons and measurements).
FUSED_ROWS = True
_mlp_slices: dict[tuple, int] = {}


def mlp_fused_slice(rows: int, hidden: int, inner: int, norm: bool, dtype: torch.dtype) -> int:
    """How wide a slice of the inner width a block of the fused feed-forward kernel takes for
    these sizes; 0 when that kernel does not take them (more than 16 rows, a 32-bit model, a
    width whose slices do not fit shared memory) or is switched off."""
    if not FUSED_ROWS or dtype != torch.bfloat16 or rows > 16:
        return 0
    key = (rows, hidden, inner, norm)
    got = _mlp_slices.get(key)
    if got is None:
        got = _mlp_slices[key] = int(_lib().rl_mlp_fused_slice(rows, hidden, inner, int(norm)))
    return got


def mlp_pack_out_weight(w_out: torch.Tensor, slice_width: int) -> torch.Tensor:
    """``w_out`` [hidden, inner] as the fused feed-forward kernel reads it: [slices, hidden,
    slice_width + 8], slice s holding ``w_out[:, s*slice_width : (s+1)*slice_width]`` followed by
    eight zero columns (the padding its rows have in shared memory), units beyond ``inner`` zero.
    A block then fetches its slice with one copy instead of one per row."""
    hidden, inner = w_out.shape
    n = -(-inner // slice_width)
    wide = torch.zeros(hidden, n * slice_width, dtype=w_out.dtype, device=w_out.device)
    wide[:, :inner] = w_out
    packed = torch.zeros(n, hidden, slice_width + 8, dtype=w_out.dtype, device=w_out.device)
    packed[:, :, :slice_width] = wide.view(hidden, n, slice_width).permute(1, 0, 2)
    return packed.contiguous()


def mlp_fused(x, h, w_in, b_in, w_out_packed, b_out, *, act: int, slice_width: int) -> None:
    """x += act(h @ w_in.T + b_in) @ w_out.T + b_out for at most 16 rows, in one kernel.

    x float32 [rows, hidden] (the residual stream); ``h`` the bfloat16 input rows, or a
    ``NormInput`` over ``x`` itself (the kernel then normalises the rows); w_in [inner, hidden]
    bfloat16; ``w_out_packed``: ``mlp_pack_out_weight(w_out, slice_width)``; biases float32 or
    ``None``.  ``slice_width``: what ``mlp_fused_slice`` returned.  The sum over slices of the inner width is taken with
    float32 atomic additions: its order, and so its last bits, may differ from run to run.
    """
    _need(x, "x", torch.float32, contiguous=False)
    _need(w_in, "w_in", torch.bfloat16)
    _need(w_out_packed, "w_out_packed", torch.bfloat16)
    rows, hidden = x.shape
    inner = w_in.shape[0]
    if w_in.shape[1] != hidden or slice_width <= 0 \
            or tuple(w_out_packed.shape) != (-(-inner // slice_width), hidden, slice_width + 8):
        raise KernelError(f"mlp_fused: weights {tuple(w_in.shape)} and (packed) {tuple(w_out_packed.shape)} do not fit "
                          f"rows of {hidden} and slices of {slice_width}")
    norm = h if isinstance(h, NormInput) else None
    if norm is not None:
        if norm.x.data_ptr() != x.data_ptr() or norm.x.stride(0) != x.stride(0):
            raise KernelError("mlp_fused: the fused norm reads the residual stream it adds to")
        a_ptr, lda, gamma, beta, eps = None, 0, norm.gamma.data_ptr(), _ptr(norm.beta), norm.eps
    else:
        _need(h, "h", torch.bfloat16, contiguous=False)
        if tuple(h.shape) != (rows, hidden) or h.stride(1) != 1:
            raise KernelError("mlp_fused: input rows do not fit the residual stream")
        a_ptr, lda, gamma, beta, eps = h.data_ptr(), h.stride(0), None, None, 0.0
    for b, n, name in ((b_in, inner, "b_in"), (b_out, hidden, "b_out")):
        if b is not None:
            _need(b, name, torch.float32)
            if b.numel() != n:
                raise KernelError(f"mlp_fused: {name} has {b.numel()} entries, not {n}")
    rc = _lib().rl_mlp_fused(x.data_ptr(), x.stride(0), a_ptr, lda, gamma, beta, eps, w_in.data_ptr(), _ptr(b_in),
                             w_out_packed.data_ptr(), _ptr(b_out), rows, hidden, inner, slice_width, act,
                             _ptr(status_word(x.device)), _stream())
    if rc == -2:
        raise KernelError(f"mlp_fused: sizes not taken (rows {rows}, hidden {hidden}, inner {inner}, slice {slice_width})")
    _ok(rc, "mlp_fused")


_attn_block_fits: dict[tuple, bool] = {}


def attn_block_fused_fits(rows: int, hidden: int, n_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the fused attention kernel of a decode step (csrc/attn_block_fused.cu) takes these
    sizes: bfloat16, at most 16 rows, hidden = heads x head size up to 1024, head size 16, 32, 64
    or 128, and a grid (heads x up to 8 blocks) that the device holds at once."""
    if not FUSED_ROWS or dtype != torch.bfloat16 or rows > 16:
        return False
    key = (rows, hidden, n_heads, head_dim)
    got = _attn_block_fits.get(key)
    if got is None:
        got = _attn_block_fits[key] = bool(_lib().rl_attn_block_fused_fits(rows, hidden, n_heads, head_dim))
    return got


def attn_block_fused_cluster(hidden: int, n_heads: int, head_dim: int, dtype: torch.dtype) -> int:
    """Blocks that share a head in the fused attention kernel at these sizes (0: not taken)."""
    if dtype != torch.bfloat16:
        return 0
    return int(_lib().rl_attn_block_fused_cluster(hidden, n_heads, head_dim))


def attn_pack_out_weight(w_out: torch.Tensor, n_heads: int, head_dim: int, cluster: int) -> torch.Tensor:
    """``w_out`` [hidden, hidden] as the fused attention kernel reads it: [heads, cluster, NO,
    head_dim + 8] with NO = hidden / cluster rounded up to a multiple of 8; slice (h, c) holds
    ``w_out[c*NO : (c+1)*NO, h*head_dim : (h+1)*head_dim]`` (rows beyond hidden zero) followed by
    eight zero columns, the padding its rows have in shared memory."""
    hidden = w_out.shape[0]
    no = -(-(hidden // 8) // cluster) * 8
    tall = torch.zeros(cluster * no, hidden, dtype=w_out.dtype, device=w_out.device)
    tall[:hidden] = w_out
    packed = torch.zeros(n_heads, cluster, no, head_dim + 8, dtype=w_out.dtype, device=w_out.device)
    packed[..., :head_dim] = tall.view(cluster, no, n_heads, head_dim).permute(2, 0, 1, 3)
    return packed.contiguous()


def attn_block_fused(x, norm: NormInput, w_qkv, b_qkv, w_out_packed, b_out, pool, block_table, positions, slots, *,
                     n_heads: int, scale: float, max_pos: int) -> None:
    """x += (attention of LayerNorm(x) over the cache) @ w_out.T + b_out, for a step in which every
    row is the new token of a decoded request (row r: request r, at ``positions[r]``, block-table
    row ``slots[r]``; a negative slot marks a padding row).  The new keys and values are written
    to their pages.  One kernel; the keys below each request's new position must be of earlier
    steps, and the sum over heads is taken with float32 atomic additions, in no fixed order.
    ``w_out_packed``: ``attn_pack_out_weight(w_out, ...)``."""
    _need(x, "x", torch.float32, contiguous=False)
    _need(w_qkv, "w_qkv", torch.bfloat16)
    _need(w_out_packed, "w_out_packed", torch.bfloat16)
    _need(pool, "pool", torch.bfloat16)
    rows, hidden = x.shape
    _, two, n_kv, page_size, dh = pool.shape
    if norm.x.data_ptr() != x.data_ptr() or norm.x.stride(0) != x.stride(0):
        raise KernelError("attn_block_fused: the fused norm reads the residual stream it adds to")
    if n_kv != n_heads or n_heads * dh != hidden or tuple(w_qkv.shape) != (3 * hidden, hidden):
        raise KernelError("attn_block_fused: as many key/value heads as heads, hidden = heads x head size")
    cluster = attn_block_fused_cluster(hidden, n_heads, dh, torch.bfloat16)
    if cluster == 0 or tuple(w_out_packed.shape) != (n_heads, cluster, -(-(hidden // 8) // cluster) * 8, dh + 8):
        raise KernelError("attn_block_fused: the output matrix is not laid out for these sizes (attn_pack_out_weight)")
    for b, n, name in ((b_qkv, 3 * hidden, "b_qkv"), (b_out, hidden, "b_out")):
        if b is not None:
            _need(b, name, torch.float32)
            if b.numel() != n:
                raise KernelError(f"attn_block_fused: {name} has {b.numel()} entries, not {n}")
    _need(positions, "positions", torch.int32)
    _need(slots, "slots", torch.int32)
    if positions.numel() < rows or slots.numel() < rows:
        raise KernelError("attn_block_fused: a position and a slot for every row")
    rc = _lib().rl_attn_block_fused(x.data_ptr(), x.stride(0), norm.gamma.data_ptr(), _ptr(norm.beta), norm.eps,
                                    w_qkv.data_ptr(), _ptr(b_qkv), w_out_packed.data_ptr(), _ptr(b_out), pool.data_ptr(),
                                    block_table.data_ptr(), block_table.stride(0), positions.data_ptr(),
                                    slots.data_ptr(), rows, hidden, n_heads, dh, page_size, max_pos, float(scale),
                                    _ptr(status_word(x.device)), _stream())
    if rc == -2:
        raise KernelError(f"attn_block_fused: sizes not taken (rows {rows}, hidden {hidden}, heads {n_heads} of {dh})")
    _ok(rc, "attn_block_fused")


def kv_write(k, v, pool, block_table, positions, req_of_token, slots, max_pos: int) -> None:
    """Copy the step's keys and values [tokens, kv heads*head dim] (views with a row stride)
    into the pages ``block_table[slots[req_of_token[n]]][positions[n] // page]``."""
    _need(k, "k", contiguous=False)
    _need(v, "v", k.dtype, contiguous=False)
    _need(pool, "pool", k.dtype)
    _need(block_table, "block_table", torch.int32)
    n_tokens = k.shape[0]
    _, two, n_kv, page_size, dh = pool.shape
    if two != 2 or k.shape[1] != n_kv * dh or k.stride(1) != 1 or v.stride(1) != 1 or k.stride(0) != v.stride(0):
        raise KernelError("kv_write: keys/values do not fit the pool")
    if dh % 16 != 0:
        raise KernelError(f"kv_write: head size {dh} is not a multiple of 16")
    if k.data_ptr() % 16 or v.data_ptr() % 16 or k.stride(0) % 8:
        raise KernelError("kv_write: key and value rows must start on 16-byte boundaries")
    rc = _lib().rl_kv_write(_code(k), _ptr(k), _ptr(v), k.stride(0), _ptr(pool), _ptr(block_table),
                            block_table.stride(0), _ptr(positions), _ptr(req_of_token), _ptr(slots),
                            n_tokens, n_kv, dh, page_size, block_table.shape[1] * page_size,
                            _ptr(status_word(k.device)), _stream())
    _ok(rc, "kv_write")


def attention(q, pool, block_table, q_start, kv_len, slots, out, *, n_heads: int, scale: float,
              window: int | None, tiles, n_tiles: int, decode_reqs, n_decode: int,
              n_splits: int = 1, part_o=None, part_ml=None, tiles_wide=None, n_tiles_wide: int = 0,
              decode_wide: bool = False, prefill_path: str | None = None, old_keys_settled: bool = False) -> None:
    """Causal attention of the step's queries over the paged cache (see csrc/attention.cu).

    q [tokens, heads*head dim] (a view with a row stride), out the same shape; ``tiles``
    int32 [n_tiles, 2] lists (request, first query) of 16-query tiles of prompt portions,
    ``decode_reqs`` int32 [n_decode] the requests with one query.  ``tiles_wide``: the
    portions again as 64-query tiles, used instead of ``tiles`` by the tensor-core kernel
    (bfloat16, head size up to 128).  ``decode_wide``: the blocks of decoded requests have
    sixteen warps instead of four (few requests, so that their keys need no split).
    ``prefill_path`` (for tests): ``"tc"`` or ``"mma"`` forces the kernel of the prompt portions.
    ``old_keys_settled``: the caller promises that the block table and the keys and values below
    each decoded request's last position were written by work that was over before the kernel
    preceding this call on the stream began (true inside the engine, whose steps are separated
    by a copy to the device); the decode kernel then fetches them before it waits for the
    kernels ahead of it.  Off, it reads nothing before that wait, and a cache write issued just
    before this call is seen.
    """
    _need(q, "q", contiguous=False)
    _need(pool, "pool", q.dtype)
    _need(out, "out", q.dtype, contiguous=False)
    _, two, n_kv, page_size, dh = pool.shape
    if dh % 16 != 0 or dh > 256:
        raise KernelError(f"attention: head size {dh} must be a multiple of 16, at most 256")
    if n_heads % n_kv != 0:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {n_kv} key/value heads")
    if q.shape[1] != n_heads * dh or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention: q does not fit heads * head size")
    if n_splits > 1:
        need = n_decode * n_heads * n_splits
        if part_o is None or part_ml is None or part_o.numel() < need * dh or part_ml.numel() < need * 2:
            raise KernelError("attention: scratch for the split partial results is too small")
        _need(part_o, "part_o", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
    rc = _lib().rl_attention(_code(q), _ptr(q), q.stride(0), _ptr(pool), _ptr(block_table), block_table.stride(0),
                             _ptr(q_start), _ptr(kv_len), _ptr(slots), _ptr(out), out.stride(0),
                             n_heads, n_kv, dh, page_size, int(window or 0), float(scale),
                             _ptr(tiles), n_tiles, _ptr(tiles_wide), n_tiles_wide if tiles_wide is not None else 0,
                             _ptr(decode_reqs), n_decode, n_splits, int(decode_wide),
                             _ptr(part_o), _ptr(part_ml), q.shape[0], pool.shape[0],
                             {None: 0, "mma": 1, "tc": 2}[prefill_path], int(old_keys_settled),
                             _ptr(status_word(q.device)), _stream())
    if rc == -5:
        raise KernelError("attention: the tcgen05 kernel takes bfloat16, head size 64, no window and pages of "
                          "8 to 128 tokens that divide 128")
    _ok(rc, "attention")
    global _launches
    _launches += (1 if n_tiles and n_decode else 0) + (1 if n_decode and n_splits > 1 else 0)


def sample(logits, temperature, top_k, top_p, seeds, counters, out_ids, kept=None, filtered: bool | None = None) -> None:
    """One token per row of float32 logits.  Rows with temperature <= 0 take the arg-max.

    temperature float32, top_k int32 (0: off), top_p float32 (>= 1: off), seeds int64,
    counters int32 (index of the generated token within its request), out_ids int32.
    ``filtered``: whether any row has top-k or top-p switched on (``None``: not known; the
    kernel for such rows is then launched whenever ``top_k`` or ``top_p`` is given).
    """
    _need(logits, "logits", torch.float32, contiguous=False)
    if logits.stride(1) != 1:
        raise KernelError("sample: rows of logits must be contiguous")
    n, vocab = logits.shape
    for t, name, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                        (top_p, "top_p", torch.float32), (seeds, "seeds", torch.int64),
                        (counters, "counters", torch.int32)):
        if t is not None:
            _need(t, name, dt)
            if t.numel() < n:
                raise KernelError(f"sample: {name} is shorter than the number of rows")
    if temperature is not None and (seeds is None or counters is None):
        raise KernelError("sample: sampling rows need seeds and counters")
    _need(out_ids, "out_ids", torch.int32)
    n_chunks = SAMPLE_CHUNKS if vocab >= 4096 else 1
    part = tickets = None
    if n_chunks > 1:
        part, tickets = _sample_scratch(logits.device, n)
    rc = _lib().rl_sample(_ptr(logits), logits.stride(0), n, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p),
                          _ptr(seeds), _ptr(counters), _ptr(out_ids), _ptr(kept), n_chunks, _ptr(part),
                          _ptr(tickets), int(filtered is None or bool(filtered)), _stream())
    _ok(rc, "sample")


# Blocks that share a row of a large vocabulary in the sampling kernel.
SAMPLE_CHUNKS = 32
_sample_bufs: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


def _sample_scratch(device: torch.device, rows: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Partial winners and tickets of the sampling kernel; the tickets are zero between calls."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    have = _sample_bufs.get(key)
    if have is None or have[1].numel() < rows:
        cap = max(256, rows)
        have = (torch.empty(cap * SAMPLE_CHUNKS * 2, dtype=torch.float32, device=device),
                torch.zeros(cap, dtype=torch.int32, device=device))
        _sample_bufs[key] = have
    return have


# ---- RMS norm --------------------------------------------------------------------------------

def rmsnorm(x, gamma, eps: float, out, rows=None) -> None:
    """out[i] = x[rows[i]] (or x[i]) / sqrt(mean(x^2) + eps) * gamma; x float32 (rows may be a
    view with a row stride), out float32 or bfloat16."""
    _need(x, "x", torch.float32, contiguous=False)
    _need(gamma, "gamma", torch.float32)
    _need(out, "out", contiguous=False)
    n_out, width = out.shape
    if x.stride(1) != 1 or out.stride(1) != 1 or x.shape[1] != width or gamma.numel() != width:
        raise KernelError("rmsnorm: widths differ, or rows are not contiguous")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        if rows.numel() < n_out:
            raise KernelError("rmsnorm: rows shorter than out")
    elif x.shape[0] < n_out:
        raise KernelError("rmsnorm: x has fewer rows than out")
    _ok(_lib().rl_rmsnorm(_code(out), _ptr(x), x.stride(0), _ptr(rows), _ptr(gamma), _ptr(out), out.stride(0), n_out,
                          width, float(eps), _stream()), "rmsnorm")


def rmsnorm_add(y, gamma, eps: float, stream_rows, mult: float, copy=None) -> None:
    """stream_rows += mult * y / sqrt(mean(y^2) + eps) * gamma (all float32); ``copy`` (bfloat16,
    same shape) receives the rounded new rows of the stream."""
    _need(y, "y", torch.float32, contiguous=False)
    _need(gamma, "gamma", torch.float32)
    _need(stream_rows, "stream_rows", torch.float32, contiguous=False)
    n, width = stream_rows.shape
    if tuple(y.shape) != (n, width) or gamma.numel() != width or y.stride(1) != 1 or stream_rows.stride(1) != 1:
        raise KernelError("rmsnorm_add: shapes differ")
    if copy is not None:
        _need(copy, "copy", torch.bfloat16, contiguous=False)
        if tuple(copy.shape) != (n, width) or copy.stride(1) != 1:
            raise KernelError("rmsnorm_add: the copy has another shape")
    _ok(_lib().rl_rmsnorm_add(_ptr(y), y.stride(0), _ptr(gamma), _ptr(stream_rows), stream_rows.stride(0), _ptr(copy),
                              0 if copy is None else copy.stride(0), n, width, float(eps), float(mult), _stream()),
        "rmsnorm_add")


def cast_rows(x, out) -> None:
    """out = bfloat16(x), both contiguous and of one shape."""
    _need(x, "x", torch.float32)
    _need(out, "out", torch.bfloat16)
    if x.numel() != out.numel():
        raise KernelError("cast_rows: sizes differ")
    _ok(_lib().rl_cast_rows(_ptr(x), _ptr(out), x.numel(), _stream()), "cast_rows")


# ---- attention over a cache of latents -----------------------------------------------------------

def latent_attention_fits(n_heads: int, rank: int, row_width: int) -> bool:
    return bool(_lib().rl_latent_attention_fits(n_heads, rank, row_width))


def latent_decode_fits(n_heads: int, rank: int, row_width: int) -> bool:
    """Whether decoded requests can take the kernel that serves all heads of a request in one block."""
    return bool(_lib().rl_latent_decode_fits(n_heads, rank, row_width))


def latent_kv_write(dkv, gamma, eps: float, inv_freq, rot_dims: int, pool, block_table, positions, req_of_token, slots,
                    *, rank: int, rot_dim: int, max_pos: int, rot_mult: float = 1.0) -> None:
    """The step's cache rows: ``dkv`` float32 [tokens, rank + rot_dim]; the first ``rank`` entries
    RMS-normalised (``gamma``, ``eps``), the next ``rot_dim`` rotated by the token's position in
    their first ``rot_dims`` entries (pairs (2i, 2i+1), angle position * inv_freq[i]); written to
    ``pool`` [pages, 1, 1, page size, row width] in the pool's dtype, zeros beyond.  ``rot_mult``: a factor of the
    cosines and sines."""
    _need(dkv, "dkv", torch.float32, contiguous=False)
    _need(gamma, "gamma", torch.float32)
    _need(pool, "pool")
    _need(block_table, "block_table", torch.int32)
    n_pages, planes, heads, page_size, row_width = pool.shape
    if planes != 1 or heads != 1 or dkv.shape[1] < rank + rot_dim or dkv.stride(1) != 1 or gamma.numel() != rank:
        raise KernelError("latent_kv_write: the pool holds one row a token; dkv holds the latent and the rotated part")
    if rot_dims:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() < rot_dims // 2:
            raise KernelError("latent_kv_write: a frequency for every rotated pair")
    rc = _lib().rl_latent_kv_write(_code(pool), _ptr(dkv), dkv.stride(0), _ptr(gamma), float(eps), _ptr(inv_freq),
                                   rot_dims, _ptr(pool), _ptr(block_table), block_table.stride(0), _ptr(positions),
                                   _ptr(req_of_token), _ptr(slots), dkv.shape[0], rank, rot_dim, row_width, page_size,
                                   max_pos, float(rot_mult), _ptr(status_word(pool.device)), _stream())
    _ok(rc, "latent_kv_write")


def latent_q_rope(q, rows, inv_freq, positions, *, n_heads: int, head_in: int, plain: int, rank: int, rot_dim: int,
                  rot_dims: int, row_width: int, rot_mult: float = 1.0) -> None:
    """rows[t, h, rank:row_width] = the rotated part of head h's query (q[t, h*head_in + plain:
    ... + rot_dim]) turned by positions[t], then zeros."""
    _need(q, "q", contiguous=False)
    _need(rows, "rows", q.dtype, contiguous=False)
    n = q.shape[0]
    if q.shape[1] != n_heads * head_in or rows.shape[1] != n_heads * row_width or q.stride(1) != 1 or rows.stride(1) != 1:
        raise KernelError("latent_q_rope: widths do not fit the heads")
    rc = _lib().rl_latent_q_rope(_code(q), _ptr(q), q.stride(0), head_in, plain, _ptr(rows), rows.stride(0), row_width,
                                 rank, rot_dim, rot_dims, _ptr(inv_freq), _ptr(positions), n, n_heads, float(rot_mult),
                                 _stream())
    _ok(rc, "latent_q_rope")


def latent_attention(q, pool, block_table, q_start, kv_len, slots, out, *, sink, n_heads: int, rank: int, scale: float,
                     tiles, n_tiles: int, decode_reqs, n_decode: int, decode_by_request: bool = False,
                     n_splits: int = 1, part_o=None, part_ml=None, simt_only: bool = False) -> None:
    """Causal attention of the step's query rows ``q`` [tokens, heads * row width] over the cached
    latent rows (``pool`` [pages, 1, 1, page size, row width]); a row's first ``rank`` entries are
    its value; ``out`` [tokens, heads * rank].  ``sink`` float32 [heads] or ``None``.
    ``decode_by_request``: decoded requests take the kernel that serves all heads in one block
    and cuts a request's keys into ``n_splits`` parts (scratch ``part_o``, ``part_ml``).  bfloat16
    runs on the tensor cores where the sizes fit and decoded requests go by request;
    ``simt_only`` (for tests and comparisons) keeps it on the CUDA-core kernels."""
    _need(q, "q", contiguous=False)
    _need(pool, "pool", q.dtype)
    _need(out, "out", q.dtype, contiguous=False)
    _, planes, heads, page_size, row_width = pool.shape
    if planes != 1 or heads != 1 or q.shape[1] != n_heads * row_width or out.shape[1] != n_heads * rank:
        raise KernelError("latent_attention: shapes do not fit the pool")
    if sink is not None:
        _need(sink, "sink", torch.float32)
        if sink.numel() != n_heads:
            raise KernelError("latent_attention: a sink per head")
    if decode_by_request and n_splits > 1:
        need = n_decode * n_heads * n_splits
        if part_o is None or part_ml is None or part_o.numel() < need * rank or part_ml.numel() < need * 2:
            raise KernelError("latent_attention: scratch for the split partial results is too small")
    rc = _lib().rl_latent_attention(_code(q), _ptr(q), q.stride(0), _ptr(pool), _ptr(block_table), block_table.stride(0),
                                    _ptr(q_start), _ptr(kv_len), _ptr(slots), _ptr(out), out.stride(0), _ptr(sink),
                                    n_heads, rank, row_width, page_size, float(scale), _ptr(tiles), n_tiles,
                                    _ptr(decode_reqs), n_decode, int(decode_by_request), n_splits, _ptr(part_o),
                                    _ptr(part_ml), int(simt_only), _ptr(status_word(q.device)), _stream())
    if rc in (-2, -3):
        raise KernelError(f"latent_attention: sizes not taken (heads {n_heads}, value width {rank}, row width {row_width})")
    _ok(rc, "latent_attention")
    global _launches
    if decode_by_request and n_decode:
        _launches += (1 if n_tiles else 0) + (1 if n_splits > 1 else 0)


def head_linear(inp, w, out, *, n_tokens: int, n_heads: int, k: int, n: int, in_strides, w_strides, out_strides,
                gate=None, gate_strides=(0, 0)) -> None:
    """out[t, h, :n] = inp[t, h, :k] @ W_h for every head: element (t, h, i) of ``inp`` at
    ``t*in_strides[0] + h*in_strides[1] + i``, element (h, i, j) of ``w`` at ``h*w_strides[0] +
    i*w_strides[1] + j*w_strides[2]``, element (t, h, j) of ``out`` at ``t*out_strides[0] +
    h*out_strides[1] + j`` (strides in elements; the tensors give base addresses and dtype).  ``gate``: float32
    logits, element (t, h, j) at ``t*gate_strides[0] + h*gate_strides[1] + j``: the result times their sigmoid."""
    _need(inp, "inp", contiguous=False)
    _need(w, "w", inp.dtype)
    _need(out, "out", inp.dtype, contiguous=False)
    if gate is not None:
        _need(gate, "gate", torch.float32, contiguous=False)
    rc = _lib().rl_head_linear(_code(inp), _ptr(inp), in_strides[0], in_strides[1], _ptr(w), w_strides[0], w_strides[1],
                               w_strides[2], _ptr(out), out_strides[0], out_strides[1], n_tokens, n_heads, k, n,
                               _ptr(gate), gate_strides[0], gate_strides[1], _stream())
    _ok(rc, "head_linear")


# ---- gated feed-forward, token-gated input, mixture of experts ---------------------------------

GATES = {"relu": 0, "silu": 1, "gelu_tanh": 2, "clamped_swish": 3}


def gated_act(gu, out, *, width: int, up_at: int, gate: int, alpha: float = 1.0, limit: float = 0.0) -> None:
    """out[r, f] = f(gu[r, f], gu[r, up_at + f]) for f < width (see csrc/gated_act.cuh)."""
    _need(gu, "gu", contiguous=False)
    _need(out, "out", gu.dtype, contiguous=False)
    if gu.shape[1] < up_at + width or out.shape[1] < width or out.shape[0] != gu.shape[0]:
        raise KernelError("gated_act: shapes do not fit")
    _ok(_lib().rl_gated_act(_code(gu), _ptr(gu), gu.stride(0), up_at, _ptr(out), out.stride(0), gu.shape[0], width,
                            gate, float(alpha), float(limit), _stream()), "gated_act")


def gate_mul(o, g) -> None:
    """o <- o * sigmoid(g) in place: ``o`` [rows, width] float32 or bfloat16, ``g`` float32 logits of the same shape;
    both may be views with a row stride."""
    _need(o, "o", contiguous=False)
    _need(g, "g", torch.float32, contiguous=False)
    if tuple(o.shape) != tuple(g.shape) or o.stride(1) != 1 or g.stride(1) != 1:
        raise KernelError("gate_mul: shapes differ, or rows are not contiguous")
    _ok(_lib().rl_gate_mul(_code(o), _ptr(o), o.stride(0), _ptr(g), g.stride(0), o.shape[0], o.shape[1], _stream()), "gate_mul")


def stream_inject(x, vec=None, again=None, keep=None, norm=None) -> None:
    """``keep <- x`` (where given), then ``x <- x + vec + again``: ``x``, ``again``, ``keep`` float32 [rows, width],
    ``vec`` float32 [width] added to every row; any of the three may be ``None``.  ``norm``: ``(gamma, eps, out)``:
    the same launch leaves ``out = x / sqrt(mean(x^2) + eps) * gamma`` of the new rows (float32 or bfloat16)."""
    _need(x, "x", torch.float32, contiguous=False)
    n, width = x.shape
    if vec is not None:
        _need(vec, "vec", torch.float32)
        if vec.numel() != width:
            raise KernelError("stream_inject: the row to add has another width")
    for t, name in ((again, "again"), (keep, "keep")):
        if t is not None:
            _need(t, name, torch.float32, contiguous=False)
            if tuple(t.shape) != (n, width) or t.stride(1) != 1:
                raise KernelError(f"stream_inject: {name} has another shape")
    if x.stride(1) != 1 or (again is not None and keep is not None and again.data_ptr() == keep.data_ptr()):
        raise KernelError("stream_inject: rows must be contiguous, and the rows kept are not the rows added")
    if norm is not None:
        gamma, eps, out = norm
        _need(gamma, "gamma", torch.float32)
        _need(out, "out", contiguous=False)
        if gamma.numel() != width or tuple(out.shape) != (n, width) or out.stride(1) != 1:
            raise KernelError("stream_inject: the norm's weight or output has another shape")
        _ok(_lib().rl_stream_inject_norm(_code(out), _ptr(x), x.stride(0), _ptr(vec), _ptr(again),
                                         0 if again is None else again.stride(0), _ptr(keep),
                                         0 if keep is None else keep.stride(0), _ptr(gamma), float(eps), _ptr(out),
                                         out.stride(0), n, width, _stream()), "stream_inject (with the norm)")
        return
    _ok(_lib().rl_stream_inject(_ptr(x), x.stride(0), _ptr(vec), _ptr(again), 0 if again is None else again.stride(0),
                                _ptr(keep), 0 if keep is None else keep.stride(0), n, width, _stream()), "stream_inject")


def token_gate(s, token_ids, table, col0: int, dim: int, out, feedback=None) -> None:
    """out[n, j] = gelu_tanh(s[n, j]) * table[token_ids[n], col0 + j] for j < dim, zero beyond."""
    _need(s, "s", contiguous=False)
    _need(table, "table", s.dtype)
    _need(out, "out", s.dtype, contiguous=False)
    _need(token_ids, "token_ids", torch.int32)
    if s.shape[1] < dim or out.shape[0] != s.shape[0] or col0 + dim > table.shape[1]:
        raise KernelError("token_gate: shapes do not fit")
    rc = _lib().rl_token_gate(_code(s), _ptr(s), s.stride(0), _ptr(token_ids), _ptr(table), table.stride(0), col0, dim,
                              _ptr(out), out.stride(0), out.shape[1], s.shape[0], table.shape[0], _ptr(feedback),
                              0 if feedback is None else feedback.numel(), _ptr(status_word(s.device)), _stream())
    _ok(rc, "token_gate")


def moe_max_tiles(n_pairs: int, n_experts: int) -> int:
    return int(_lib().rl_moe_max_tiles(n_pairs, n_experts))


MOE_SCORES = {"softmax": 0, "sigmoid": 1}


def moe_select(z, correction, *, top: int, group_count: int, group_keep: int, ids, weights, counts,
               score: int = 0) -> None:
    """Routing of every row of the float32 router logits ``z`` [tokens, experts]: see csrc/moe.cu.
    ``ids`` int32 and ``weights`` float32 [tokens * top]; ``counts`` int32 [experts], zero on entry.
    ``score``: 0 softmax over the experts, 1 each expert's sigmoid."""
    _need(z, "z", torch.float32, contiguous=False)
    n, n_experts = z.shape
    for t, name, dt in ((ids, "ids", torch.int32), (weights, "weights", torch.float32), (counts, "counts", torch.int32)):
        _need(t, name, dt)
    if correction is not None:
        _need(correction, "correction", torch.float32)
    rc = _lib().rl_moe_select(_ptr(z), z.stride(0), _ptr(correction), n, n_experts, top, group_count, group_keep,
                              int(score), _ptr(ids), _ptr(weights), _ptr(counts), _stream())
    if rc in (-2, -3):
        raise KernelError(f"moe_select: {n_experts} experts, top {top}, {group_keep} of {group_count} groups not taken")
    _ok(rc, "moe_select")


def moe_table_select(token_ids, table, *, n_experts: int, weight: float, ids, weights, counts, feedback=None) -> None:
    """Routing by a table: row ``token_ids[t]`` of ``table`` (int32 [vocab, top]) names token t's experts, each with
    ``weight``.  ``ids``, ``weights``, ``counts`` as ``moe_select`` leaves them (``counts`` zero on entry)."""
    _need(token_ids, "token_ids", torch.int32)
    _need(table, "table", torch.int32)
    for t, name, dt in ((ids, "ids", torch.int32), (weights, "weights", torch.float32), (counts, "counts", torch.int32)):
        _need(t, name, dt)
    vocab, top = table.shape
    n = token_ids.numel()
    if ids.numel() < n * top or weights.numel() < n * top or counts.numel() < n_experts:
        raise KernelError("moe_table_select: the outputs are too small")
    rc = _lib().rl_moe_table_select(_ptr(token_ids), _ptr(table), vocab, n, n_experts, top, float(weight), _ptr(ids),
                                    _ptr(weights), _ptr(counts), _ptr(feedback), 0 if feedback is None else feedback.numel(),
                                    _ptr(status_word(table.device)), _stream())
    if rc == -2:
        raise KernelError(f"moe_table_select: {n_experts} experts, {top} a token not taken")
    _ok(rc, "moe_table_select")


MOE_TABLE_ROUTE_MAX_PAIRS = 8192  # csrc/moe.cu: MOE_ROUTE_MAX_PAIRS


def moe_table_route(token_ids, table, *, n_experts: int, weight: float, ids, weights, offsets, tiles, meta, row_token,
                    place_of, feedback=None) -> None:
    """``moe_table_select`` and ``moe_plan`` in one launch, for at most ``MOE_TABLE_ROUTE_MAX_PAIRS`` (token, choice)
    pairs: the same ``ids``, ``weights``, ``offsets``, ``tiles``, ``meta``, ``row_token`` and ``place_of``."""
    _need(token_ids, "token_ids", torch.int32)
    _need(table, "table", torch.int32)
    _need(weights, "weights", torch.float32)
    for t, name in ((ids, "ids"), (offsets, "offsets"), (tiles, "tiles"), (meta, "meta"), (row_token, "row_token"),
                    (place_of, "place_of")):
        _need(t, name, torch.int32)
    vocab, top = table.shape
    n = token_ids.numel()
    if min(ids.numel(), weights.numel(), row_token.numel(), place_of.numel()) < n * top or offsets.numel() < n_experts + 1 \
            or tiles.numel() < 3 * moe_max_tiles(n * top, n_experts):
        raise KernelError("moe_table_route: the outputs are too small")
    rc = _lib().rl_moe_table_route(_ptr(token_ids), _ptr(table), vocab, n, n_experts, top, float(weight), _ptr(ids),
                                   _ptr(weights), _ptr(offsets), _ptr(tiles), _ptr(meta), _ptr(row_token), _ptr(place_of),
                                   _ptr(feedback), 0 if feedback is None else feedback.numel(),
                                   _ptr(status_word(table.device)), _stream())
    if rc in (-2, -3):
        raise KernelError(f"moe_table_route: {n_experts} experts, {top} a token, {n} tokens not taken")
    _ok(rc, "moe_table_route")


def moe_plan(ids, counts, fill, offsets, tiles, meta, row_token, place_of, *, n_tokens: int, n_experts: int, top: int,
             weights=None, place_weight=None) -> None:
    """Lay the chosen pairs out expert by expert (all int32 device buffers; see csrc/moe.cu).
    With ``weights`` and ``place_weight`` (float32 [tokens * top]) the pairs' weights are left by
    place, for experts whose INPUT is weighted."""
    if (weights is None) != (place_weight is None):
        raise KernelError("moe_plan: weights and place_weight go together")
    rc = _lib().rl_moe_plan(_ptr(ids), _ptr(counts), _ptr(fill), _ptr(offsets), _ptr(tiles), _ptr(meta), _ptr(row_token),
                            _ptr(place_of), _ptr(weights), _ptr(place_weight), n_tokens, n_experts, top, _stream())
    _ok(rc, "moe_plan")
    global _launches
    _launches += 1


def moe_experts(h, w_gate_up, w_down, tiles, meta, row_token, place_of, weights, act, eo, y, *, n_experts: int, top: int,
                ff: int, gate: int, alpha: float, limit: float, add: bool, place_weight=None) -> None:
    """The experts' gated feed-forward on the laid-out pairs and the weighted sum per token into
    ``y`` float32 [tokens, hidden] (``add``: added to it).  ``weights`` (by pair) weight the experts'
    outputs; ``place_weight`` (by place, from ``moe_plan``) their inputs instead; either may be ``None``.  ``w_gate_up`` [experts * 2 * ff, hidden]
    (per expert: gate rows, then up rows), ``w_down`` [experts * hidden, ff]."""
    _need(h, "h", contiguous=False)
    _need(w_gate_up, "w_gate_up", h.dtype)
    _need(w_down, "w_down", h.dtype)
    _need(act, "act", h.dtype, contiguous=False)
    _need(eo, "eo", torch.float32)
    _need(y, "y", torch.float32, contiguous=False)
    n, hidden = h.shape
    if tuple(w_gate_up.shape) != (n_experts * 2 * ff, hidden) or tuple(w_down.shape) != (n_experts * hidden, ff) \
            or act.shape[0] < n * top or act.shape[1] < ff or eo.numel() < n * top * hidden or tuple(y.shape) != (n, hidden):
        raise KernelError("moe_experts: shapes do not fit")
    rc = _lib().rl_moe_experts(_code(h), _ptr(h), h.stride(0), _ptr(w_gate_up), _ptr(w_down), _ptr(tiles), _ptr(meta),
                               _ptr(row_token), _ptr(place_of), _ptr(weights), _ptr(place_weight), _ptr(act), act.stride(0), _ptr(eo), _ptr(y),
                               y.stride(0), n, hidden, ff, n_experts, top, gate, float(alpha), float(limit), int(add),
                               _stream())
    _ok(rc, "moe_experts")
    global _launches
    _launches += 2


# ---- embedding with a table chosen by pairs of tokens ------------------------------------------

def embed_pair(token_ids, positions, req_of_token, q_start, slots, table, pos_table, pair_table, out, last_token, *,
               buckets: int, mul_prev: int, mul_cur: int, feedback=None) -> None:
    """out[n] = table[id_n] + pair_table[(prev_n * mul_prev + id_n * mul_cur) mod buckets] (+ pos_table[pos_n]);
    a sequence's first token takes row ``buckets`` of ``pair_table``.  ``last_token`` int32 [slots, 1]:
    each request's last token so far (read for a portion's first token, then brought up to date)."""
    _need(token_ids, "token_ids", torch.int32)
    _need(positions, "positions", torch.int32)
    _need(table, "table")
    _need(pair_table, "pair_table", table.dtype)
    _need(out, "out", torch.float32)
    _need(last_token, "last_token", torch.int32)
    n, hidden = out.shape
    if table.shape[1] != hidden or pair_table.shape[1] != hidden or pair_table.shape[0] != buckets + 1:
        raise KernelError("embed_pair: table widths differ from out, or the pair table has not buckets + 1 rows")
    n_pos = 0
    if pos_table is not None:
        _need(pos_table, "pos_table", table.dtype)
        n_pos = pos_table.shape[0]
    rc = _lib().rl_embed_pair(_code(table), _ptr(token_ids), _ptr(positions), _ptr(req_of_token), _ptr(q_start),
                              _ptr(slots), _ptr(table), _ptr(pos_table), _ptr(pair_table), _ptr(out), n, hidden,
                              table.shape[0], n_pos, int(buckets), int(mul_prev), int(mul_cur), _ptr(last_token),
                              _ptr(status_word(out.device)), _ptr(feedback), 0 if feedback is None else feedback.numel(),
                              _stream())
    _ok(rc, "embed_pair")


def rmsnorm_add_norm(y, gamma, eps: float, stream_rows, gamma_next, eps_next: float, out_next) -> None:
    """stream_rows += y / sqrt(mean(y^2) + eps) * gamma, then out_next = the new rows normalised with
    ``gamma_next`` (float32 or bfloat16): the norm behind one sublayer and the norm ahead of the next in one pass."""
    _need(y, "y", torch.float32, contiguous=False)
    _need(gamma, "gamma", torch.float32)
    _need(gamma_next, "gamma_next", torch.float32)
    _need(stream_rows, "stream_rows", torch.float32, contiguous=False)
    _need(out_next, "out_next", contiguous=False)
    n, width = stream_rows.shape
    if tuple(y.shape) != (n, width) or tuple(out_next.shape) != (n, width) or gamma.numel() != width \
            or gamma_next.numel() != width or y.stride(1) != 1 or stream_rows.stride(1) != 1 or out_next.stride(1) != 1:
        raise KernelError("rmsnorm_add_norm: shapes differ")
    rc = _lib().rl_rmsnorm_add_norm(_code(out_next), _ptr(y), y.stride(0), _ptr(gamma), _ptr(stream_rows),
                                    stream_rows.stride(0), _ptr(gamma_next), _ptr(out_next), out_next.stride(0), n, width,
                                    float(eps), float(eps_next), _stream())
    if rc == -2:
        raise KernelError(f"rmsnorm_add_norm: rows of {width} elements do not fit a block's shared memory")
    _ok(rc, "rmsnorm_add_norm")


RMSNORM_ADD_NORM_MAX_WIDTH = 48 * 1024 // 4 - 64


# ---- mixers with a matrix-valued state -------------------------------------------------------------

RECURRENCES = {"delta": 0, "gated": 1, "decayed_keys": 2, "matrix_memory": 3}


def recurrence_record(mode: int, dk: int, dv: int) -> int:
    """Floats of the record that ``recurrence`` keeps per (head, token) in its ``prep`` scratch."""
    a, b, c = c_int(0), c_int(0), c_int(0)
    if _lib().rl_recurrence_record(int(mode), int(dk), int(dv), ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)) != 0:
        raise KernelError(f"recurrence: sizes not taken (key size {dk}, value size {dv}: up to 256 each)")
    return c.value


def recurrence(mode: int, proj, offsets: dict, state, out, q_start, slots, prep, oraw, *, n_reqs: int, n_heads: int,
               dk: int, dv: int, eps: float, a_bias, w0, out_weight, w2t=None, rank: int = 0, decay_scale: float = 0.0,
               unit_eps: float = 0.0, tau: float = 0.0, cap: float = 0.0, floor_eps: float = 0.0, qscale: float = 1.0,
               gates=None) -> None:
    """One step of a recurrence over matrix states (csrc/recurrent.cu) for every request of the step.
    ``proj`` float32 [tokens, columns]: the packed projections, ``offsets`` the first column of
    ``r``, ``k``, ``v``, ``a``, ``g``, ``w`` (those the form has); ``state`` float32
    [slots, heads, dk, dv]; ``out`` [tokens, heads * dv] float32 or bfloat16; ``prep`` float32 scratch of
    heads * tokens * ``recurrence_record`` floats, ``oraw`` float32 scratch [tokens, heads * dv];
    ``w2t`` float32 [rank, heads * dk]: the low-rank decay's second matrix, transposed.
    The matrix memory (mode 3) keeps its normaliser as one more column of the state and a running maximum a
    head behind the matrices: ``state`` float32 [slots, heads * dk * (dv + 1) + heads]; ``gates`` float32 scratch
    of tokens * heads * 4 floats; ``cap`` bounds the gates' logits, ``floor_eps`` is added to the output's divisor;
    ``a_bias`` / ``w0`` are the input and forget gates' biases [heads].  ``tau`` (mode 2): the decay is
    sigmoid(.)^(1/tau); ``qscale`` (modes 2, 3) multiplies the queries."""
    _need(proj, "proj", torch.float32, contiguous=False)
    _need(state, "state", torch.float32)
    _need(out, "out", contiguous=False)
    _need(prep, "prep", torch.float32)
    _need(oraw, "oraw", torch.float32)
    for t, name in ((a_bias, "a_bias"), (w0, "w0"), (out_weight, "out_weight")):
        _need(t, name, torch.float32)
    n_tokens = proj.shape[0]
    if w2t is not None:
        _need(w2t, "w2t", torch.float32)
        if tuple(w2t.shape) != (rank, n_heads * dk):
            raise KernelError("recurrence: the low-rank matrix has another shape")
    dvs = dv + 1 if mode == 3 else dv  # columns of a head's state
    want_state = (n_heads * dk * dvs + n_heads,) if mode == 3 else (n_heads, dk, dv)
    if tuple(state.shape[1:]) != want_state or out.shape[1] != n_heads * dv or proj.stride(1) != 1 \
            or out.stride(1) != 1 or out.shape[0] != n_tokens:
        raise KernelError("recurrence: shapes do not fit")
    if prep.numel() < n_heads * n_tokens * recurrence_record(mode, dk, dvs) or oraw.numel() < n_tokens * n_heads * dvs:
        raise KernelError("recurrence: scratch too small")
    if mode == 2 and (w2t is None or rank <= 0 or tau <= 0):
        raise KernelError("recurrence: the form with decaying key channels needs its low-rank decay and tau")
    if mode == 3:
        if gates is None or gates.dtype != torch.float32 or gates.numel() < n_tokens * n_heads * 4 or cap <= 0:
            raise KernelError("recurrence: the matrix memory needs its gates' scratch and a positive cap")
    if mode == 0 and (w2t is None or rank <= 0):
        raise KernelError("recurrence: the delta form needs its low-rank decay")
    off = [int(offsets.get(k, -1)) for k in ("r", "k", "v", "a", "g", "w")]
    rc = _lib().rl_recurrence(int(mode), _code(out), _ptr(proj), proj.stride(0), *off, _ptr(a_bias), _ptr(w0), _ptr(w2t),
                              int(rank), _ptr(out_weight), _ptr(state), _ptr(out), out.stride(0), _ptr(q_start),
                              _ptr(slots), _ptr(prep), _ptr(oraw), n_tokens, n_reqs, n_heads, dk, dvs, float(eps),
                              float(decay_scale), float(unit_eps), state.stride(0), n_heads * dk * dvs, float(tau),
                              float(cap), float(floor_eps), float(qscale), _ptr(gates), _stream())
    if rc == -2:
        raise KernelError(f"recurrence: sizes not taken (key size {dk}, value size {dv}: up to 256 each)")
    _ok(rc, "recurrence")
    global _launches
    _launches += 3 if mode == 3 else 2


# ---- attention with a distance bias over rows of [key | value] -------------------------------------

BIAS_ATTENTION_TENSOR_CORES = True  # prompt portions in bfloat16 on mma.sync (off: the CUDA-core kernel throughout)


def bias_attention_tensor_cores(dtype: torch.dtype, dk: int, dv: int) -> bool:
    """Whether ``bias_attention`` may be asked for its tensor-core form for prompt portions."""
    return BIAS_ATTENTION_TENSOR_CORES and dtype == torch.bfloat16 and dk <= 128 and dv <= 128


def bias_attention_async(on: bool) -> None:
    """For comparisons and tests: let the tensor-core prompt tiles take the form whose key and value tiles travel
    by cp.async through a ring of two stages (the default, where cache rows can be copied in 16-byte pieces), or
    keep every size on the form that copies them through registers."""
    lib = _lib()
    lib.rl_bias_attention_async.argtypes = [c_int]
    lib.rl_bias_attention_async.restype = None
    lib.rl_bias_attention_async(int(bool(on)))


def bias_attention_shape(heads_per_group: int, tensor_cores: bool = False) -> tuple[int, int]:
    """(heads a block, tokens a block) of ``bias_attention``'s prompt tiles for so many query heads a
    key/value head: of the 32 rows of the CUDA-core kernel's blocks, or the 64 of the tensor-core kernel's."""
    hb, tt = c_int(0), c_int(0)
    if _lib().rl_bias_attention_shape(int(heads_per_group), 64 if tensor_cores else 32, ctypes.byref(hb), ctypes.byref(tt)) != 0:
        raise KernelError("bias_attention_shape: heads per group must be positive")
    return hb.value, tt.value


def bias_kv_store(k, v, pool, block_table, positions, req_of_token, slots, *, v_at: int, max_pos: int, mix: int = 0,
                  v_src=None, lam=None) -> None:
    """The step's keys ``k`` [tokens, kv heads * dk] and values ``v`` [tokens, kv heads * dv] (float32 views)
    into the pool [pages, 1, kv heads, page, row], the value at entry ``v_at`` of a row.  ``mix`` 1: the
    values are also left in ``v_src`` (float32 [tokens, kv heads * dv]); 2: v <- (1 - lam) v + lam v_src
    (``lam`` a float32 device scalar) goes into the pages."""
    _need(k, "k", torch.float32, contiguous=False)
    _need(v, "v", torch.float32, contiguous=False)
    _need(pool, "pool")
    n = k.shape[0]
    _, planes, n_kv, page_size, row = pool.shape
    dk, dv = k.shape[1] // n_kv, v.shape[1] // n_kv
    if planes != 1 or k.shape[1] != n_kv * dk or v.shape[1] != n_kv * dv or v.shape[0] != n:
        raise KernelError("bias_kv_store: shapes do not fit the pool")
    if v_src is not None:
        _need(v_src, "v_src", torch.float32)
        if v_src.numel() < n * n_kv * dv:
            raise KernelError("bias_kv_store: the value source is too small")
    if lam is not None:
        _need(lam, "lam", torch.float32)
    rc = _lib().rl_bias_kv_store(_code(pool), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(v_src), _ptr(lam), int(mix),
                                 _ptr(pool), _ptr(block_table), block_table.stride(0), _ptr(positions), _ptr(req_of_token),
                                 _ptr(slots), n, n_kv, dk, dv, int(v_at), row, page_size,
                                 min(block_table.shape[1], -(-max_pos // page_size)), _ptr(status_word(pool.device)),
                                 _stream())
    if rc == -2:
        raise KernelError("bias_kv_store: the mixing mode lacks its buffers, or the value does not fit the row")
    _ok(rc, "bias_kv_store")


def bias_attention(q, gate, pool, block_table, q_start, kv_len, slots, out, *, n_heads: int, dk: int, dv: int, v_at: int,
                   scale: float, slopes=None, temp_coef: float = 0.0, temp_every: int = 0, tiles=None, n_tiles: int = 0,
                   tile_tokens: int = 16, decode_reqs=None, n_decode: int = 0, max_pos: int, n_splits: int = 1, part_o=None,
                   part_ml=None, tensor_cores: bool = False, window: int = 0, head_scale=None, sink=None,
                   gate_per_head: bool = False) -> None:
    """Causal attention of the step's queries over the cached rows (csrc/bias_attention.cu).
    ``tensor_cores``: prompt portions on mma.sync (bfloat16 pool and output, sizes up to 128; the tiles cut as
    ``bias_attention_shape(.., True)`` says).
    ``n_splits`` > 1: the keys of every decoded request are cut into so many parts (``part_o`` float32
    [n_decode * heads * n_splits, dv] and ``part_ml`` [.., 2] are their scratch) and merged in order.
    ``q`` float32 [tokens, heads * dk] and ``gate`` float32 [tokens, heads * dv] (or ``None``) may be views
    with a row stride; ``out`` [tokens, heads * dv] float32 or bfloat16; ``slopes`` float32 [heads] or ``None``.
    ``window`` > 0: a query sees itself and the ``window - 1`` keys before it; ``head_scale`` float32 [heads]: a
    further factor of every score of a head; ``sink`` float32 [heads]: one more term exp(sink[h]) in the softmax's
    denominator (no key, no value, not scaled); ``gate_per_head``: ``gate`` is [tokens, heads], one logit a head."""
    _need(q, "q", torch.float32, contiguous=False)
    _need(out, "out", contiguous=False)
    _need(pool, "pool")
    _, planes, n_kv, page_size, row = pool.shape
    if planes != 1 or q.shape[1] != n_heads * dk or out.shape[1] != n_heads * dv or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("bias_attention: shapes do not fit")
    if gate is not None:
        _need(gate, "gate", torch.float32, contiguous=False)
        if gate.shape[1] != (n_heads if gate_per_head else n_heads * dv) or gate.stride(1) != 1:
            raise KernelError("bias_attention: the gate has another shape")
    for t, name in ((slopes, "slopes"), (head_scale, "head_scale"), (sink, "sink")):
        if t is not None:
            _need(t, name, torch.float32)
            if t.numel() != n_heads:
                raise KernelError(f"bias_attention: {name} has one entry a head")
    global _launches
    if n_decode <= 0:
        n_splits = 1
    if n_splits > 1:
        if part_o is None or part_ml is None or part_o.dtype != torch.float32 or part_ml.dtype != torch.float32 \
                or part_o.numel() < n_decode * n_heads * n_splits * dv or part_ml.numel() < n_decode * n_heads * n_splits * 2:
            raise KernelError("bias_attention: the parts' scratch is missing or too small")
        _launches += 1
    rc = _lib().rl_bias_attention(_code(pool), _code(out), _ptr(q), q.stride(0), _ptr(gate), 0 if gate is None else gate.stride(0),
                                  _ptr(pool), _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(kv_len),
                                  _ptr(slots), _ptr(tiles), int(n_tiles), int(tile_tokens), _ptr(decode_reqs), int(n_decode),
                                  _ptr(out), out.stride(0), n_heads, n_kv, dk, dv, int(v_at), row, page_size,
                                  min(block_table.shape[1], -(-max_pos // page_size)), float(scale), float(temp_coef),
                                  int(temp_every), _ptr(slopes), _ptr(status_word(out.device)), int(n_splits), _ptr(part_o),
                                  _ptr(part_ml), int(bool(tensor_cores) and bias_attention_tensor_cores(pool.dtype, dk, dv)
                                                     and out.dtype == torch.bfloat16), int(window), _ptr(head_scale),
                                  _ptr(sink), int(bool(gate_per_head)), _stream())
    if rc in (-2, -3, -4):
        raise KernelError(f"bias_attention: sizes not taken (code {rc}: key and value sizes up to 256; tiles a multiple "
                          "of the tokens a block takes)")
    _ok(rc, "bias_attention")


class QkvCache:
    """Where ``qkv_norm_rotate`` puts the step's keys and values: the pool ``[pages, 1, kv heads, page, row]`` (the
    value at entry ``v_at`` of a row), the block table and the step's request and slot arrays."""

    def __init__(self, pool, block_table, req_of_token, slots, v_at: int, max_pos: int) -> None:
        self.pool, self.block_table, self.req_of_token, self.slots = pool, block_table, req_of_token, slots
        self.v_at, self.max_pos = int(v_at), int(max_pos)


def qkv_norm_rotate(q, k, v, positions, *, n_heads: int, n_kv: int, dk: int, dv: int, eps: float, q_norm=None, k_norm=None,
                    freq=None, rot_dims: int = 0, unit_values: bool = False, unit_qk: bool = False,
                    cache: "QkvCache | None" = None) -> None:
    """In place on float32 views (row strides allowed): every head of ``q`` [tokens, heads * dk] and ``k``
    [tokens, kv heads * dk] divided by its root mean square and multiplied by ``q_norm`` / ``k_norm`` (float32
    [dk], both or neither), then its first ``rot_dims`` entries turned in neighbouring pairs by position *
    ``freq[i]``; with ``unit_values`` every head of ``v`` [tokens, kv heads * dv] divided by its root mean square;
    with ``unit_qk`` (and no weights) every head of q and k divided by its root mean square and left so.
    ``cache`` (a ``QkvCache``): keys and values go into their cache pages as ``bias_kv_store`` would put them (and
    are not written back in place): no store kernel is needed behind this one."""
    for t, name, width in ((q, "q", n_heads * dk), (k, "k", n_kv * dk), (v, "v", n_kv * dv)):
        _need(t, name, torch.float32, contiguous=False)
        if t.shape[1] != width or t.stride(1) != 1 or t.shape[0] != q.shape[0]:
            raise KernelError(f"qkv_norm_rotate: {name} has another shape")
    for t, name in ((q_norm, "q_norm"), (k_norm, "k_norm")):
        if t is not None:
            _need(t, name, torch.float32)
            if t.numel() != dk:
                raise KernelError(f"qkv_norm_rotate: {name} has one entry a key channel")
    if rot_dims:
        _need(freq, "freq", torch.float32)
        if freq.numel() < rot_dims // 2:
            raise KernelError("qkv_norm_rotate: one frequency a turned pair")
    cx = (0, None, None, 0, None, None, 0, 0, 0, 0, None)
    if cache is not None:
        pool = cache.pool
        _need(pool, "cache.pool")
        _need(cache.block_table, "cache.block_table", torch.int32)
        _, planes, heads, page_size, row = pool.shape
        if planes != 1 or heads != n_kv or cache.v_at < dk or cache.v_at + dv > row:
            raise KernelError("qkv_norm_rotate: the cache's rows do not fit the keys and values")
        cx = (_code(pool), _ptr(pool), _ptr(cache.block_table), cache.block_table.stride(0), _ptr(cache.req_of_token),
              _ptr(cache.slots), int(cache.v_at), row, page_size,
              min(cache.block_table.shape[1], -(-cache.max_pos // page_size)), _ptr(status_word(pool.device)))
    rc = _lib().rl_qkv_norm_rotate(_ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(q_norm), _ptr(k_norm),
                                   _ptr(freq) if rot_dims else None, _ptr(positions), q.shape[0], n_heads, n_kv, dk, dv,
                                   int(rot_dims), int(bool(unit_values)), int(bool(unit_qk)), float(eps), *cx, _stream())
    if rc == -2:
        raise KernelError("qkv_norm_rotate: sizes not taken (an even number of turned entries, at most the key size; "
                          "both norms or neither)")
    _ok(rc, "qkv_norm_rotate")


def gated_join_norm(y0, s0: float, y1, s1: float, z, gamma, eps: float, alpha: float, stream_rows, copy=None,
                    z_bias=None) -> None:
    """stream = rmsnorm(alpha * stream + sigmoid(z + z_bias) * (s0 * y0 + s1 * y1)) * gamma, row by row in float32
    (``y1`` may be ``None``; ``z`` ``None``: no gate; ``z_bias`` float32 [width] or ``None``); ``copy`` (bfloat16, or
    ``None``) receives the new rows rounded."""
    n, width = stream_rows.shape
    _need(stream_rows, "stream_rows", torch.float32)
    _need(gamma, "gamma", torch.float32)
    for t, name in ((y0, "y0"), (y1, "y1"), (z, "z")):
        if t is None and name != "y0":
            continue
        _need(t, name, torch.float32, contiguous=False)
        if tuple(t.shape) != (n, width) or t.stride(1) != 1:
            raise KernelError(f"gated_join_norm: {name} has another shape")
    if gamma.numel() != width:
        raise KernelError("gated_join_norm: the norm's weight has another size")
    if z_bias is not None:
        _need(z_bias, "z_bias", torch.float32)
        if z_bias.numel() != width or z is None:
            raise KernelError("gated_join_norm: the gate's bias has one entry a column, and needs the gate's logits")
    if copy is not None:
        _need(copy, "copy", torch.bfloat16)
        if tuple(copy.shape) != (n, width):
            raise KernelError("gated_join_norm: the copy has another shape")
    rc = _lib().rl_gated_join_norm(_ptr(y0), y0.stride(0), float(s0), _ptr(y1), 0 if y1 is None else y1.stride(0), float(s1),
                                   _ptr(z), 0 if z is None else z.stride(0), _ptr(z_bias), _ptr(gamma), _ptr(stream_rows), stream_rows.stride(0), _ptr(copy),
                                   0 if copy is None else copy.stride(0), n, width, float(eps), float(alpha), _stream())
    _ok(rc, "gated_join_norm")
