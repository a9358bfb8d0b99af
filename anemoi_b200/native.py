"""ctypes binding of ``libanemoi_sm100.so`` (the C ABI declared in include/anemoi_sm100.h).

Plays the role of the reference's backend wrappers over ``torch.ops.mixed_attention.*``
(anemoi/layers/attention/mpa/backends/sm120_q64.py, sm120_q128.py, sm89_k64.py and
mpa/build_identity.py): one Python function per native entry point, marshaling
tensors to raw device pointers on the current CUDA stream.  There is no fallback:
a missing library raises.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from functools import lru_cache
from pathlib import Path

import torch

LIBRARY_NAME = "libanemoi_sm100.so"

(BUF_Q_FP16, BUF_KV_FP16, BUF_Q_INT8, BUF_KV_INT8, BUF_Q_NVFP4, BUF_KV_NVFP4, BUF_Q_INT8_SCALE,
 BUF_K_INT8_SCALE, BUF_V_E4M3_SCALE, BUF_V_AMAX, BUF_POOL, BUF_COUNT) = range(12)

ERRORS = {-1: "invalid argument", -2: "CUDA launch failure", -3: "size beyond a documented limit"}

# Kernels of this library launched so far by the calling process, per entry point (each wrapper
# below adds what its entry launches; memset nodes are not kernels).  Benchmarks read the
# difference over their timed region.
LAUNCHES: dict[str, int] = {}


def _count(name: str, kernels: int) -> None:
    LAUNCHES[name] = LAUNCHES.get(name, 0) + kernels


def launches_total() -> int:
    return sum(LAUNCHES.values())


class Shape(C.Structure):
    _fields_ = [
        ("heads", C.c_int32), ("head_dim", C.c_int32), ("query_block", C.c_int32),
        ("seq_tokens", C.c_int32), ("prefix_tokens", C.c_int32), ("video_blocks", C.c_int32),
        ("has_nvfp4", C.c_int32), ("has_int8", C.c_int32), ("has_fp16", C.c_int32),
        ("has_prefix_query_int8", C.c_int32), ("has_maxpool", C.c_int32),
        ("input_is_bf16", C.c_int32),
        ("q_global_scale", C.c_float), ("k_global_scale", C.c_float), ("v_global_scale", C.c_float),
    ]

    @property
    def prefix_stages(self) -> int:
        return math.ceil(self.prefix_tokens / 64)

    @property
    def stages(self) -> int:
        return self.prefix_stages + self.video_blocks * (self.query_block // 64)

    @property
    def prefix_query_tiles(self) -> int:
        if not self.has_prefix_query_int8:
            return 0
        return math.ceil(self.prefix_tokens / self.query_block)


class Operands(C.Structure):
    _fields_ = [(name, C.c_void_p) for name in (
        "q_fp16", "kv_fp16", "q_int8", "kv_int8", "q_nvfp4", "kv_nvfp4", "q_int8_scale",
        "k_int8_scale", "v_e4m3_scale", "v_amax", "q_pool", "k_pool", "q_max_pool", "k_max_pool")]


@lru_cache(maxsize=1)
def library() -> C.CDLL:
    """Load the in-tree shared library; raise if it has not been built."""
    path = Path(__file__).resolve().parent / LIBRARY_NAME
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m anemoi_b200.build` "
            "(nvcc, sm_100a). There is no fallback path."
        )
    lib = C.CDLL(str(path))
    P, I32, I64, F = C.c_void_p, C.c_int32, C.c_int64, C.c_float
    SP, OP = C.POINTER(Shape), C.POINTER(Operands)
    signatures = {
        "anemoi_sm100_arch": (C.c_int, []),
        "anemoi_sm100_operand_bytes": (I64, [SP, C.c_int]),
        "anemoi_sm100_prepare": (C.c_int, [SP, P, P, P, C.POINTER(I64), P, P, OP, P]),
        "anemoi_sm100_draft_probability": (C.c_int, [SP, P, P, P, P, F, P, P]),
        "anemoi_sm100_draft_probability_jensen": (C.c_int, [SP, P, P, P, P, P, P]),
        "anemoi_sm100_route_scratch_bytes": (I64, [SP]),
        "anemoi_sm100_route_list_capacity": (I64, [SP, I64, I64, I64, C.c_int]),
        "anemoi_sm100_route": (C.c_int, [SP, P, I64, I64, I64, C.c_int, P, I64, P, P, P, I64, P]),
        "anemoi_sm100_route_static_max_bytes": (I64, []),
        "anemoi_sm100_route_anchored_scratch_bytes": (I64, [SP]),
        "anemoi_sm100_route_anchored": (C.c_int, [SP, P, I64, I64, I64, C.c_int, P, P, I32, P, I64, P, P, P, I64, P]),
        "anemoi_sm100_route_static": (C.c_int, [SP, P, I64, I64, I64, C.c_int, P, P, P, I64, P]),
        "anemoi_sm100_attention": (C.c_int, [SP, OP, P, P, P, I64, P, P, P, P]),
        "anemoi_sm100_attention_pairs": (C.c_int, [SP, OP, P, P, P, P, I64, P, P, P, P]),
        "anemoi_sm100_pair_lists": (C.c_int, [SP, P, P, P, I64, P, P, P]),
        "anemoi_sm100_prefix_attention": (C.c_int, [SP, OP, P, P, P, P]),
        "anemoi_sm100_copy_rows": (C.c_int, [P, I64, P, I64, I64, I64, I32, P]),
        "anemoi_sm100_peer_alloc": (C.c_int, [I64, C.POINTER(P), P]),
        "anemoi_sm100_peer_open": (C.c_int, [P, C.POINTER(P)]),
        "anemoi_sm100_peer_close": (C.c_int, [P]),
        "anemoi_sm100_peer_free": (C.c_int, [P]),
        "anemoi_sm100_push_qkv": (C.c_int, [P, P, P, C.POINTER(P), C.POINTER(P), C.POINTER(I64), I32, I32, I32,
                                            I32, C.POINTER(I64), C.c_uint32, P, P]),
        "anemoi_sm100_push_qkv_norm": (C.c_int, [P, P, P, P, P, P, P, I32, C.c_float, I32, C.POINTER(P),
                                                 C.POINTER(P), C.POINTER(I64), I32, I32, I32, I32,
                                                 C.POINTER(I64), C.c_uint32, P, P]),
        "anemoi_sm100_push_out": (C.c_int, [P, C.POINTER(P), C.POINTER(P), C.POINTER(I64), I32, I32, I32, I32,
                                            C.c_uint32, P, P]),
        "anemoi_sm100_wait_flags": (C.c_int, [P, I32, C.c_uint32, C.c_uint64, P, P]),
        "anemoi_sm100_set_wait_limit_ns": (C.c_int, [C.c_uint64]),
        "anemoi_sm100_wait_selftest": (C.c_int, [C.c_uint64, P, P]),
        "anemoi_sm100_assemble": (C.c_int, [SP, P, I64, C.c_int, P, P, P, P, P]),
        "anemoi_sm100_pack_qkv": (C.c_int, [P, P, P, P, I64, I32, I32, I32, C.POINTER(I64), P]),
        "anemoi_sm100_merge_heads": (C.c_int, [P, P, I64, I32, I32, I32, P]),
        "anemoi_sm100_pack_qkv_heads": (C.c_int, [P, P, P, P, I64, I32, I32, I32, I32, I32,
                                                  C.POINTER(C.c_int64), P]),
        "anemoi_sm100_merge_heads_into": (C.c_int, [P, P, I64, I32, I32, I32, I32, I32, P]),
        "anemoi_sm100_tensor_peak": (C.c_int, [I32, I32, P, C.POINTER(C.c_double), P]),
        "anemoi_sm100_qknorm_rope": (C.c_int, [P, P, P, P, I64, I32, I32, I32, C.c_float, I32,
                                               C.POINTER(C.c_int64), P]),
    }
    for name, (restype, argtypes) in signatures.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.anemoi_sm100_arch() != 100:
        raise RuntimeError("libanemoi_sm100.so was not built for sm_100a")
    return lib


EXPORTED = (
    "anemoi_sm100_arch", "anemoi_sm100_operand_bytes", "anemoi_sm100_prepare",
    "anemoi_sm100_draft_probability", "anemoi_sm100_draft_probability_jensen", "anemoi_sm100_route_scratch_bytes",
    "anemoi_sm100_route_list_capacity", "anemoi_sm100_route", "anemoi_sm100_route_static",
    "anemoi_sm100_route_static_max_bytes", "anemoi_sm100_attention",
    "anemoi_sm100_attention_pairs", "anemoi_sm100_pair_lists",
    "anemoi_sm100_route_anchored", "anemoi_sm100_route_anchored_scratch_bytes",
    "anemoi_sm100_prefix_attention", "anemoi_sm100_assemble", "anemoi_sm100_pack_qkv",
    "anemoi_sm100_merge_heads", "anemoi_sm100_pack_qkv_heads", "anemoi_sm100_merge_heads_into",
    "anemoi_sm100_tensor_peak", "anemoi_sm100_qknorm_rope", "anemoi_sm100_set_wait_limit_ns",
    "anemoi_sm100_wait_selftest", "anemoi_sm100_copy_rows", "anemoi_sm100_push_qkv",
    "anemoi_sm100_push_qkv_norm", "anemoi_sm100_push_out", "anemoi_sm100_wait_flags", "anemoi_sm100_peer_alloc", "anemoi_sm100_peer_open",
    "anemoi_sm100_peer_close", "anemoi_sm100_peer_free",
)


def _check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed: {ERRORS.get(code, code)}")


def _ptr(t: torch.Tensor | None):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


@dataclass
class OperandStore:
    """Device buffers behind an ``Operands`` struct (kept alive with it)."""

    shape: Shape
    buffers: dict
    struct: Operands

    def raw(self, name: str) -> torch.Tensor:
        return self.buffers[name]


def allocate_operands(shape: Shape, device) -> OperandStore:
    lib = library()

    def nbytes(which: int) -> int:
        n = lib.anemoi_sm100_operand_bytes(C.byref(shape), which)
        if n < 0:
            raise RuntimeError("invalid attention shape")
        return int(n)

    buffers: dict[str, torch.Tensor | None] = {}

    def alloc(name: str, which: int, dtype=torch.uint8):
        n = nbytes(which)
        if n == 0:
            buffers[name] = None
            return
        itemsize = torch.empty((), dtype=dtype).element_size()
        buffers[name] = torch.empty(n // itemsize, dtype=dtype, device=device)

    alloc("q_fp16", BUF_Q_FP16)
    alloc("kv_fp16", BUF_KV_FP16)
    alloc("q_int8", BUF_Q_INT8)
    alloc("kv_int8", BUF_KV_INT8)
    alloc("q_nvfp4", BUF_Q_NVFP4)
    alloc("kv_nvfp4", BUF_KV_NVFP4)
    alloc("q_int8_scale", BUF_Q_INT8_SCALE, torch.float32)
    alloc("k_int8_scale", BUF_K_INT8_SCALE, torch.float32)
    alloc("v_e4m3_scale", BUF_V_E4M3_SCALE, torch.float32)
    alloc("v_amax", BUF_V_AMAX, torch.float32)
    pool = (shape.heads, shape.video_blocks, shape.head_dim)
    buffers["q_pool"] = torch.empty(pool, dtype=torch.float16, device=device)
    buffers["k_pool"] = torch.empty(pool, dtype=torch.float16, device=device)
    if shape.has_maxpool:
        buffers["q_max_pool"] = torch.empty(pool, dtype=torch.float16, device=device)
        buffers["k_max_pool"] = torch.empty(pool, dtype=torch.float16, device=device)
    else:
        buffers["q_max_pool"] = buffers["k_max_pool"] = None
    struct = Operands(**{k: (None if v is None else v.data_ptr()) for k, v in buffers.items()})
    return OperandStore(shape=shape, buffers=buffers, struct=struct)


def prepare(shape: Shape, q, k, v, indices, counts, store: OperandStore) -> None:
    """Fill the operand store from raw ``[1, S, H, D]`` Q/K/V views (see anemoi_sm100_prepare)."""
    strides = (C.c_int64 * 6)(q.stride(1), q.stride(2), k.stride(1), k.stride(2), v.stride(1), v.stride(2))
    _count("prepare", 2 if shape.has_int8 else 1)      # V amax pre-pass + the fused pass
    _check(library().anemoi_sm100_prepare(C.byref(shape), _ptr(q), _ptr(k), _ptr(v), strides,
                                          _ptr(indices), _ptr(counts), C.byref(store.struct),
                                          _stream(q.device)), "anemoi_sm100_prepare")


def draft_probability(shape: Shape, store: OperandStore, maxpool_weight: float) -> torch.Tensor:
    r = shape.video_blocks
    prob = torch.empty((shape.heads, r, r), dtype=torch.float16, device=store.buffers["q_pool"].device)
    b = store.buffers
    _count("draft_probability", 1)
    _check(library().anemoi_sm100_draft_probability(
        C.byref(shape), _ptr(b["q_pool"]), _ptr(b["k_pool"]), _ptr(b["q_max_pool"]),
        _ptr(b["k_max_pool"]), float(maxpool_weight), _ptr(prob), _stream(prob.device)),
        "anemoi_sm100_draft_probability")
    return prob


def draft_probability_jensen(shape: Shape, store: OperandStore) -> torch.Tensor:
    """The diag-Jensen draft map; the operands' extra pool slots hold the second moments
    (``shape.has_maxpool == 2``)."""
    if shape.has_maxpool != 2:
        raise ValueError("the operands were not prepared with second moments")
    b = store.buffers
    r = shape.video_blocks
    prob = torch.empty((shape.heads, r, r), dtype=torch.float16, device=b["q_pool"].device)
    _count("draft", 1)
    _check(library().anemoi_sm100_draft_probability_jensen(
        C.byref(shape), _ptr(b["q_pool"]), _ptr(b["k_pool"]), _ptr(b["q_max_pool"]), _ptr(b["k_max_pool"]),
        _ptr(prob), _stream(prob.device)), "anemoi_sm100_draft_probability_jensen")
    return prob


@dataclass
class RouteLists:
    row_offset: torch.Tensor   # int32 [H, R]
    row_counts: torch.Tensor   # int32 [H, R, 4]
    stage_ids: torch.Tensor    # int32 [H, capacity]
    capacity: int


def route(shape: Shape, prob: torch.Tensor, n16: int, n8: int, n4: int, prefix_phase: int) -> RouteLists:
    lib = library()
    dev = prob.device
    h, r = shape.heads, shape.video_blocks
    scratch = torch.empty(int(lib.anemoi_sm100_route_scratch_bytes(C.byref(shape))), dtype=torch.uint8,
                          device=dev)
    if not shape.prefix_tokens:
        prefix_phase = -1
    cap = int(lib.anemoi_sm100_route_list_capacity(C.byref(shape), n16, n8, n4, prefix_phase))
    lists = RouteLists(
        row_offset=torch.empty((h, r), dtype=torch.int32, device=dev),
        row_counts=torch.empty((h, r, 4), dtype=torch.int32, device=dev),
        stage_ids=torch.empty((h, max(cap, 1)), dtype=torch.int32, device=dev),
        capacity=max(cap, 1),
    )
    _count("route", 5)                                  # hist, threshold, rowstat, headscan, emit
    _check(lib.anemoi_sm100_route(C.byref(shape), _ptr(prob), n16, n8, n4, prefix_phase,
                                  _ptr(scratch), scratch.numel(), _ptr(lists.row_offset),
                                  _ptr(lists.row_counts), _ptr(lists.stage_ids), lists.capacity,
                                  _stream(dev)), "anemoi_sm100_route")
    return lists


def route_anchored(shape: Shape, prob: torch.Tensor, n16: int, n8: int, n4: int, prefix_phase: int,
                   anchors: torch.Tensor, anchor_ids: torch.Tensor) -> RouteLists:
    """Routing with anchors: ``anchors`` ``(R, R)`` bool / uint8 mask shared by the heads,
    ``anchor_ids`` its set flat indices (int32)."""
    lib = library()
    dev = prob.device
    h, r = shape.heads, shape.video_blocks
    if anchors.shape != (r, r) or anchors.dtype not in (torch.bool, torch.uint8) or anchor_ids.dtype != torch.int32:
        raise ValueError("anchors must be an (R, R) bool mask and anchor_ids int32")
    lowest = n4 or n8 or n16
    if anchor_ids.numel() > lowest:
        raise ValueError("anchor_count exceeds the configured lowest-precision budget")
    scratch = torch.empty(int(lib.anemoi_sm100_route_anchored_scratch_bytes(C.byref(shape))), dtype=torch.uint8,
                          device=dev)
    if not shape.prefix_tokens:
        prefix_phase = -1
    cap = int(lib.anemoi_sm100_route_list_capacity(C.byref(shape), n16, n8, n4, prefix_phase))
    lists = RouteLists(
        row_offset=torch.empty((h, r), dtype=torch.int32, device=dev),
        row_counts=torch.empty((h, r, 4), dtype=torch.int32, device=dev),
        stage_ids=torch.empty((h, max(cap, 1)), dtype=torch.int32, device=dev),
        capacity=max(cap, 1),
    )
    mask = anchors.contiguous().view(torch.uint8)
    _count("route", 9)     # hist, anchor hist, 2 x threshold, rowstat, tie scan, count, offsets, emit
    _check(lib.anemoi_sm100_route_anchored(
        C.byref(shape), _ptr(prob), n16, n8, n4, prefix_phase, _ptr(mask), _ptr(anchor_ids),
        int(anchor_ids.numel()), _ptr(scratch), scratch.numel(), _ptr(lists.row_offset),
        _ptr(lists.row_counts), _ptr(lists.stage_ids), lists.capacity, _stream(dev)),
        "anemoi_sm100_route_anchored")
    return lists


def route_static(shape: Shape, prob: torch.Tensor, n16: int, n8: int, n4: int, prefix_phase: int,
                 lists: RouteLists) -> None:
    """Routing into caller-owned ``lists`` with the library's built-in scratch array.

    For hosts that may not allocate on their request path: nothing is allocated here or in
    the library.  All calls on a device share one scratch array, so keep them on one stream
    (or order them with events); the first call on a device should precede stream capture."""
    if not shape.prefix_tokens:
        prefix_phase = -1
    _check(library().anemoi_sm100_route_static(
        C.byref(shape), _ptr(prob), n16, n8, n4, prefix_phase, _ptr(lists.row_offset),
        _ptr(lists.row_counts), _ptr(lists.stage_ids), lists.capacity, _stream(prob.device)),
        "anemoi_sm100_route_static")


@dataclass
class PairLists:
    """Union lists of the Q64 query-block pairs (2t, 2t+1) of every head."""
    pair_counts: torch.Tensor  # int32 [H, ceil(R/2), 4]: stages per phase of the union, launch order
    pair_ids: torch.Tensor     # int32 [H, capacity]: stage id | membership bits 30 (block 2t), 31 (2t+1)


def pair_lists(shape: Shape, lists: RouteLists) -> PairLists:
    """Merges the lists of query blocks 2t and 2t+1 (Q64 only) for ``attention(..., pairs=)``."""
    dev = lists.stage_ids.device
    pairs = PairLists(
        pair_counts=torch.empty((shape.heads, (shape.video_blocks + 1) // 2, 4), dtype=torch.int32, device=dev),
        pair_ids=torch.empty_like(lists.stage_ids))
    _count("pair_lists", 2)                              # merge, launch order
    _check(library().anemoi_sm100_pair_lists(
        C.byref(shape), _ptr(lists.row_offset), _ptr(lists.row_counts), _ptr(lists.stage_ids), lists.capacity,
        _ptr(pairs.pair_counts), _ptr(pairs.pair_ids), _stream(dev)), "anemoi_sm100_pair_lists")
    return pairs


def attention(shape: Shape, store: OperandStore, lists: RouteLists, valid_k: torch.Tensor,
              status: torch.Tensor, pairs: PairLists | None = None) -> torch.Tensor:
    """The video query blocks' attention.  With ``pairs`` (Q64) two query blocks share a CTA and
    walk the union of their lists; the result is the same."""
    dev = valid_k.device
    out = torch.empty((shape.heads, shape.video_blocks * shape.query_block, shape.head_dim),
                      dtype=torch.float16, device=dev)
    _count("attention", 1)
    if pairs is not None:
        _check(library().anemoi_sm100_attention_pairs(
            C.byref(shape), C.byref(store.struct), _ptr(lists.row_offset), _ptr(lists.row_counts),
            _ptr(pairs.pair_counts), _ptr(pairs.pair_ids), lists.capacity, _ptr(valid_k), _ptr(out),
            _ptr(status), _stream(dev)), "anemoi_sm100_attention_pairs")
        return out
    _check(library().anemoi_sm100_attention(
        C.byref(shape), C.byref(store.struct), _ptr(lists.row_offset), _ptr(lists.row_counts),
        _ptr(lists.stage_ids), lists.capacity, _ptr(valid_k), _ptr(out), _ptr(status),
        _stream(dev)), "anemoi_sm100_attention")
    return out


def prefix_attention(shape: Shape, store: OperandStore, valid_k: torch.Tensor,
                     status: torch.Tensor) -> torch.Tensor:
    dev = valid_k.device
    rows = shape.prefix_query_tiles * shape.query_block
    out = torch.empty((shape.heads, rows, shape.head_dim), dtype=torch.float16, device=dev)
    _count("prefix_attention", 1)
    _check(library().anemoi_sm100_prefix_attention(
        C.byref(shape), C.byref(store.struct), _ptr(valid_k), _ptr(out), _ptr(status),
        _stream(dev)), "anemoi_sm100_prefix_attention")
    return out


def copy_head_group(dst: torch.Tensor, src: torch.Tensor, stream: torch.cuda.Stream) -> None:
    """One strided copy of a head group between a pinned host tensor and a device tensor.

    ``dst`` and ``src`` are ``[1, S, heads, D]`` views with the same shape, contiguous in their
    last two dimensions; exactly one of them is on the device.  Asynchronous on ``stream``."""
    if dst.shape != src.shape or dst.dtype != src.dtype or dst.ndim != 4 or dst.size(0) != 1:
        raise ValueError("copy_head_group needs two [1, S, heads, D] views of one dtype")
    for t in (dst, src):
        if t.stride(3) != 1 or t.stride(2) != t.size(3):
            raise ValueError("copy_head_group needs views contiguous over (heads, D)")
        if t.device.type == "cpu" and not t.is_pinned():
            raise ValueError("the host side of copy_head_group must be pinned memory")
    to_device = dst.device.type == "cuda"
    if to_device == (src.device.type == "cuda"):
        raise ValueError("copy_head_group copies between the host and the device")
    size = dst.element_size()
    _check(library().anemoi_sm100_copy_rows(
        _ptr(dst), dst.stride(1) * size, _ptr(src), src.stride(1) * size,
        dst.size(2) * dst.size(3) * size, dst.size(1), int(to_device),
        C.c_void_p(stream.cuda_stream)), "anemoi_sm100_copy_rows")


def set_wait_limit_ns(limit_ns: int) -> None:
    """Limit of every bounded wait in attention kernels launched from now on (default 2 s)."""
    _check(library().anemoi_sm100_set_wait_limit_ns(int(limit_ns)), "anemoi_sm100_set_wait_limit_ns")


def wait_selftest(limit_ns: int, status: torch.Tensor) -> None:
    """Launch the one-CTA kernel whose wait must give up after ``limit_ns`` (sets ``status`` to 99)."""
    _check(library().anemoi_sm100_wait_selftest(int(limit_ns), _ptr(status), _stream(status.device)),
           "anemoi_sm100_wait_selftest")


def assemble(shape: Shape, prefix_out: torch.Tensor | None, out_packed: torch.Tensor,
             inverse: torch.Tensor, row_counts: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    dev = out_packed.device
    out = torch.empty((1, shape.seq_tokens, shape.heads, shape.head_dim), dtype=dtype, device=dev)
    caller = 0
    rows = 0
    if prefix_out is not None:
        rows = prefix_out.shape[1]
        if prefix_out.dtype not in (torch.float16, dtype):
            raise TypeError("prefix rows must be fp16 or the caller's dtype")
        caller = int(prefix_out.dtype != torch.float16)
    _count("assemble", 1)
    _check(library().anemoi_sm100_assemble(
        C.byref(shape), _ptr(prefix_out), rows, caller, _ptr(out_packed), _ptr(inverse),
        _ptr(row_counts), _ptr(out), _stream(dev)), "anemoi_sm100_assemble")
    return out


def pack_qkv_destination_major(q, k, v, world: int, head_begin: int = 0,
                               head_count: int | None = None) -> torch.Tensor:
    """``(rows, heads, D)`` x3 (strided views allowed) -> ``(world, rows, head_count, 3*D)``.

    Destination rank ``r`` gets its heads ``r*heads/world + head_begin + (0..head_count)``
    (default: all ``heads/world`` of them)."""
    rows, heads, d = q.shape
    if heads % world:
        raise ValueError(f"heads ({heads}) must divide the Ulysses degree ({world})")
    if not (q.shape == k.shape == v.shape and q.dtype == k.dtype == v.dtype):
        raise ValueError("q, k, v must share shape and dtype")
    if q.element_size() != 2 or any(t.stride(-1) != 1 for t in (q, k, v)):
        raise ValueError("pack_qkv needs 16-bit tensors with a contiguous head dimension")
    head_count = heads // world - head_begin if head_count is None else head_count
    if head_begin < 0 or head_count <= 0 or head_begin + head_count > heads // world:
        raise ValueError("head range outside the heads of a rank")
    out = torch.empty((world, rows, head_count, 3 * d), dtype=q.dtype, device=q.device)
    if out.numel() == 0:
        return out
    strides = (C.c_int64 * 6)(q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1))
    _count("pack_qkv", 1)
    _check(library().anemoi_sm100_pack_qkv_heads(_ptr(q), _ptr(k), _ptr(v), _ptr(out), rows, heads, d,
                                                 world, head_begin, head_count, strides,
                                                 _stream(q.device)),
           "anemoi_sm100_pack_qkv_heads")
    return out


def merge_heads(x: torch.Tensor, out: torch.Tensor | None = None, head_begin: int = 0) -> torch.Tensor:
    """``(world, rows, head_count, D)`` contiguous -> ``(rows, world*heads_per_rank, D)``.

    Without ``out`` the result holds exactly the given heads; with ``out`` (contiguous) the heads
    land at ``head_begin`` of every rank's ``out.size(1) // world`` heads."""
    world, rows, hc, d = x.shape
    if not x.is_contiguous() or x.element_size() != 2:
        raise ValueError("merge_heads needs a contiguous 16-bit tensor")
    if out is None:
        out = torch.empty((rows, world * hc, d), dtype=x.dtype, device=x.device)
    if (not out.is_contiguous() or out.dtype != x.dtype or out.size(0) != rows or out.size(2) != d
            or out.size(1) % world):
        raise ValueError("merge_heads: out must be contiguous (rows, world*heads_per_rank, D)")
    per_rank = out.size(1) // world
    if head_begin < 0 or head_begin + hc > per_rank:
        raise ValueError("head range outside the heads of a rank")
    if x.numel() == 0:
        return out
    _count("merge_heads", 1)
    _check(library().anemoi_sm100_merge_heads_into(_ptr(x), _ptr(out), rows, world, hc, d, per_rank,
                                                   head_begin, _stream(x.device)),
           "anemoi_sm100_merge_heads_into")
    return out


def peer_alloc(nbytes: int) -> tuple[int, bytes]:
    """A zero-filled device region of the current device and its 64-byte CUDA IPC handle."""
    ptr, handle = C.c_void_p(), C.create_string_buffer(64)
    _check(library().anemoi_sm100_peer_alloc(nbytes, C.byref(ptr), handle), "anemoi_sm100_peer_alloc")
    return int(ptr.value), handle.raw


def peer_open(handle: bytes) -> int:
    """Maps another process's region (same node) into this process; returns its address here."""
    ptr = C.c_void_p()
    _check(library().anemoi_sm100_peer_open(C.create_string_buffer(handle, 64), C.byref(ptr)),
           "anemoi_sm100_peer_open")
    return int(ptr.value)


def peer_close(ptr: int) -> None:
    _check(library().anemoi_sm100_peer_close(C.c_void_p(ptr)), "anemoi_sm100_peer_close")


def peer_free(ptr: int) -> None:
    _check(library().anemoi_sm100_peer_free(C.c_void_p(ptr)), "anemoi_sm100_peer_free")


def push_qkv(q, k, v, peer_recv, peer_flags, first_rows, rank: int, epoch: int, blocks_done,
             producer=None) -> None:
    """Store this rank's rows of ``q, k, v`` ``(rows, heads, D)`` into every rank's head-sharded
    receive buffer ``(all rows, heads/world, 3*D)`` and publish ``epoch`` in their flag words;
    ``peer_recv`` / ``peer_flags`` hold the addresses as mapped into this process.

    ``producer = (q_weight, k_weight, cos, sin, eps)`` applies the per-head RMS norm and partial
    rotary embedding of ``fused_qknorm_rope`` to q and k on the way (``cos``/``sin``: fp32
    ``(rows, rotary_dim)``); the caller's q and k are left as they are."""
    world = len(peer_recv)
    rows, heads, d = q.shape
    if rows != first_rows[rank + 1] - first_rows[rank]:
        raise ValueError("q, k, v must hold exactly this rank's rows")
    data = (C.c_void_p * world)(*peer_recv)
    flags = (C.c_void_p * world)(*peer_flags)
    first = (C.c_int64 * (world + 1))(*first_rows)
    strides = (C.c_int64 * 6)(q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1))
    _count("push_qkv", 1)
    if producer is not None:
        wq, wk, cos, sin, eps = producer
        rotary = int(cos.shape[-1])
        if (wq.dtype != q.dtype or wk.dtype != q.dtype or cos.dtype != torch.float32 or sin.dtype != torch.float32
                or not cos.is_contiguous() or not sin.is_contiguous() or cos.shape != (rows, rotary)
                or sin.shape != cos.shape or wq.numel() != d or wk.numel() != d):
            raise ValueError("producer needs (D,) weights of the tensors' dtype and contiguous fp32 "
                             "(rows, rotary_dim) cos / sin tables")
        _check(library().anemoi_sm100_push_qkv_norm(
            _ptr(q), _ptr(k), _ptr(v), _ptr(wq), _ptr(wk), _ptr(cos), _ptr(sin), rotary, float(eps),
            int(q.dtype == torch.bfloat16), data, flags, first, rank, world, heads, d, strides,
            epoch & 0xFFFFFFFF, _ptr(blocks_done), _stream(q.device)), "anemoi_sm100_push_qkv_norm")
        return
    _check(library().anemoi_sm100_push_qkv(_ptr(q), _ptr(k), _ptr(v), data, flags, first, rank, world, heads, d,
                                           strides, epoch & 0xFFFFFFFF, _ptr(blocks_done), _stream(q.device)),
           "anemoi_sm100_push_qkv")


def push_out(out_heads, peer_out, peer_flags, first_rows, rank: int, epoch: int, blocks_done) -> None:
    """Store the head-sharded result ``(all rows, heads_local, D)`` into the sequence-sharded
    output ``(its rows, world*heads_local, D)`` of the rank that owns each row and publish
    ``epoch`` in the owners' flag words."""
    world = len(peer_out)
    total, heads_local, d = out_heads.shape
    if not out_heads.is_contiguous() or total != first_rows[-1]:
        raise ValueError("push_out needs the contiguous (all rows, heads_local, D) result")
    data = (C.c_void_p * world)(*peer_out)
    flags = (C.c_void_p * world)(*peer_flags)
    first = (C.c_int64 * (world + 1))(*first_rows)
    _count("push_out", 1)
    _check(library().anemoi_sm100_push_out(_ptr(out_heads), data, flags, first, rank, world, heads_local, d,
                                           epoch & 0xFFFFFFFF, _ptr(blocks_done), _stream(out_heads.device)),
           "anemoi_sm100_push_out")


def wait_flags(flags_ptr: int, world: int, epoch: int, limit_ns: int, status, device) -> None:
    """One-warp kernel on the current stream: returns when every rank's flag has reached
    ``epoch``; past ``limit_ns`` it records 70 + rank in ``status`` instead."""
    _count("wait_flags", 1)
    _check(library().anemoi_sm100_wait_flags(C.c_void_p(flags_ptr), world, epoch & 0xFFFFFFFF, limit_ns,
                                             _ptr(status), _stream(device)), "anemoi_sm100_wait_flags")


TENSOR_KINDS = {"f16": 0, "i8": 1, "f8": 2, "nvfp4": 3}


def tensor_peak(kind: str, device=None, iterations: int = 4096, repeats: int = 3) -> float:
    """Measured tcgen05 throughput (TFLOP/s, or TOP/s for ``i8``) of one MMA kind.

    Runs the library's tensor-pipe probe (128x128 tiles, operands in shared memory, two CTAs per
    SM) ``repeats`` times after one warm-up and returns the best rate.  Measurement helper for
    the roofline denominators; it has no part in the attention path.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    lib = library()
    status = torch.zeros(1, dtype=torch.int32, device=device)
    flops = C.c_double(0.0)
    best = 0.0
    with torch.cuda.device(device):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for rep in range(repeats + 1):
            start.record()
            _check(lib.anemoi_sm100_tensor_peak(TENSOR_KINDS[kind], iterations, _ptr(status),
                                                C.byref(flops), _stream(device)),
                   "anemoi_sm100_tensor_peak")
            end.record()
            end.synchronize()
            if rep > 0:
                best = max(best, flops.value / (start.elapsed_time(end) * 1e-3) / 1e12)
    if int(status.item()) != 0:
        raise RuntimeError("anemoi_sm100_tensor_peak: a bounded wait gave up")
    return best


def qknorm_rope_(x: torch.Tensor, weight: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                 eps: float) -> torch.Tensor:
    """In place: per-head RMS norm with ``weight`` then partial rotary on ``x`` ``[tokens, heads, D]``
    (strided views with a contiguous last dimension are fine); ``cos``/``sin`` ``[tokens, rotary]``."""
    if x.ndim != 3 or x.dtype not in (torch.float16, torch.bfloat16) or x.stride(-1) != 1:
        raise ValueError("x must be [tokens, heads, D] fp16/bf16 with a contiguous head dimension")
    tokens, heads, d = x.shape
    if weight.shape != (d,) or weight.dtype != x.dtype or not weight.is_contiguous():
        raise ValueError("weight must be a contiguous [D] tensor of x's dtype")
    if cos.shape != sin.shape or cos.ndim != 2 or cos.size(0) != tokens:
        raise ValueError("cos and sin must be [tokens, rotary_dim]")
    cos = cos.to(device=x.device, dtype=torch.float32).contiguous()
    sin = sin.to(device=x.device, dtype=torch.float32).contiguous()
    strides = (C.c_int64 * 2)(x.stride(0), x.stride(1))
    _check(library().anemoi_sm100_qknorm_rope(_ptr(x), _ptr(weight), _ptr(cos), _ptr(sin), tokens, heads, d,
                                              cos.size(1), float(eps), int(x.dtype == torch.bfloat16),
                                              strides, _stream(x.device)),
           "anemoi_sm100_qknorm_rope")
    return x
