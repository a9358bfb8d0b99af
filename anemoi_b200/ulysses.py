"""Ulysses sequence<->head exchange around ``anemoi_attention`` for 1/2/4/8 B200s of one node.

Every rank holds a contiguous slice of the packed sequence with all heads.  q, k and v travel
together to head-sharded form (each rank: the whole sequence, ``heads / world`` heads), attention
runs on the local heads, and the output travels back to sequence-sharded form.  Heads are
independent in every stage of the attention path, so the sharded result is bit-identical to the
single-GPU result.

Two transports.  ``PeerExchange``: the relayout kernels store straight into the other ranks'
memory over NVLink (regions mapped with CUDA IPC) and hand over with one flag word per source
rank; no collective call, send buffer, pack or merge pass is on the per-layer path, and the
qk-norm + rotary step in front of the exchange can ride on the stores.  ``all_to_all_single``
(NCCL): pack kernel, collective, attention on strided views of the receive buffer, collective,
merge kernel, optionally pipelined by head groups.

Both follow the reference's custom Ulysses path
(anemoi/models/minimax_h3/solengine/models/minimax_h3/optimized/ulysses_custom.py:36-165,
relayout.py:83-162): packed destination-major layout, explicit row counts for uneven shards
(``tensor_split``, gathered once per group and cached).  The relayouts are CUDA kernels of this
library instead of Triton kernels, and the head-sharded receive buffer is consumed in place by
the preparation kernel (strided Q/K/V views), so no unpack pass exists.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import native
from .api import NVFP4Calibration, QuantConfig, SparseConfig, VisualLayout, anemoi_attention

_ROW_COUNTS: dict = {}


def shard_rows(total_rows: int, world: int) -> list[int]:
    """Row counts of ``torch.tensor_split(total_rows, world)``: the first ``total % world``
    ranks hold one row more."""
    base, extra = divmod(total_rows, world)
    return [base + (1 if r < extra else 0) for r in range(world)]


def row_counts(rows_local: int, group=None) -> list[int]:
    """Every rank's row count; one ``all_reduce`` per group, then cached.

    The cache key is the group (identical on every rank) and a changed local length
    raises instead of desynchronising the collective count across ranks."""
    key = id(group)
    cached = _ROW_COUNTS.get(key)
    if cached is not None:
        counts, seen = cached
        if seen != rows_local:
            raise RuntimeError(
                f"row count cached for rows_local={seen} but called with {rows_local}; "
                "call reset_row_counts() on every rank when the sequence length changes")
        return counts
    world = dist.get_world_size(group)
    device = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    buf = torch.zeros(world, dtype=torch.long, device=device)
    buf[dist.get_rank(group)] = rows_local
    dist.all_reduce(buf, group=group)
    counts = [int(c) for c in buf.tolist()]
    _ROW_COUNTS[key] = (counts, rows_local)
    return counts


def reset_row_counts() -> None:
    _ROW_COUNTS.clear()


def exchange_to_heads(q, k, v, counts, group=None, pack=native.pack_qkv_destination_major):
    """``(rows_local, H, D)`` x3 -> ``(S, H/world, 3*D)`` on every rank (one collective)."""
    world = len(counts)
    rows, heads, d = q.shape
    h_local = heads // world
    send = pack(q, k, v, world)                              # (world, rows, h_local, 3D)
    inner = h_local * 3 * d
    recv = torch.empty((sum(counts), h_local, 3 * d), dtype=q.dtype, device=q.device)
    dist.all_to_all_single(recv.view(-1), send.view(-1),
                           output_split_sizes=[c * inner for c in counts],
                           input_split_sizes=[rows * inner] * world, group=group)
    return recv


def exchange_to_sequence(out_heads, counts, rank: int, group=None, merge=native.merge_heads):
    """``(S, H/world, D)`` -> ``(rows_local, H, D)`` (one collective + one merge copy)."""
    world = len(counts)
    s, h_local, d = out_heads.shape
    rows = counts[rank]
    inner = h_local * d
    recv = torch.empty((world, rows, h_local, d), dtype=out_heads.dtype, device=out_heads.device)
    dist.all_to_all_single(recv.view(-1), out_heads.reshape(-1),
                           output_split_sizes=[rows * inner] * world,
                           input_split_sizes=[c * inner for c in counts], group=group)
    return merge(recv)


def head_groups(heads_local: int, groups: int) -> list[tuple[int, int]]:
    """``(begin, count)`` of at most ``groups`` contiguous, near-equal groups of a rank's heads."""
    groups = max(1, min(groups, heads_local))
    base, extra = divmod(heads_local, groups)
    out, begin = [], 0
    for g in range(groups):
        count = base + (1 if g < extra else 0)
        out.append((begin, count))
        begin += count
    return out


class _DeviceSpan:
    """A raw device range offered to torch through the CUDA array interface (no copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2, "strides": None}


def first_rows(counts: list[int]) -> list[int]:
    """First row of every rank's shard, with the total appended."""
    out = [0]
    for c in counts:
        out.append(out[-1] + c)
    return out


def exchange_region_layout(counts: list[int], heads: int, head_dim: int, itemsize: int = 2) -> dict:
    """Byte offsets inside a rank's exchange region; the same on every rank (the output slots are
    sized for the longest shard): flag words, the head-sharded q|k|v receive buffer, two
    sequence-sharded output slots used alternately."""
    world = len(counts)
    h_local = heads // world
    align = lambda n: (n + 255) // 256 * 256          # noqa: E731
    recv = sum(counts) * h_local * 3 * head_dim * itemsize
    out = max(counts) * heads * head_dim * itemsize
    layout = {"flags_in": 0, "flags_out": 64, "recv": 256}
    layout["out0"] = layout["recv"] + align(recv)
    layout["out1"] = layout["out0"] + align(out)
    layout["bytes"] = layout["out1"] + align(out)
    layout["recv_bytes"], layout["out_bytes"] = recv, out
    return layout


class PeerExchange:
    """The Ulysses exchange by direct stores into the peers' memory, for the ranks of one node.

    Construction is collective: every rank allocates one exchange region, the ranks swap its IPC
    handle over the process group and map each other's regions.  Per layer, ``to_heads`` stores
    this rank's rows of q, k, v into every rank's head-sharded receive buffer and returns the
    local one once all ranks' parts have landed; ``to_sequence`` stores the head-sharded result
    into the owners' output buffers and returns the local one likewise.  No collective library
    call and no send, receive or merge copy is on the per-layer path: two store kernels and two
    one-warp flag waits.  The calls must alternate (the hand-over that makes buffer reuse safe
    depends on it); the returned output view is overwritten by the second ``to_sequence`` after
    it.  A wait past ``limit_ns`` records 70 + the late rank in the device's sticky status word
    (``executor.last_status``) and the stream continues."""

    def __init__(self, rows_local: int, heads: int, head_dim: int, dtype, device, group=None,
                 limit_ns: int = 10_000_000_000):
        from .executor import _status_word

        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("the exchange carries fp16 / bf16 rows")
        self.group, self.device, self.dtype = group, torch.device(device), dtype
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if heads % self.world or self.world > 8:
            raise ValueError(f"heads ({heads}) must divide the Ulysses degree ({self.world} <= 8)")
        self.heads, self.head_dim, self.h_local = heads, head_dim, heads // self.world
        self.counts = row_counts(rows_local, group)
        self.first = first_rows(self.counts)
        self.layout = exchange_region_layout(self.counts, heads, head_dim)
        self.limit_ns = limit_ns
        self.status = _status_word(self.device)
        # set-up is collective and must not leave a rank behind: every rank reports how far it
        # got, and all of them either finish or clean up and raise together
        self.base, self.mapped, error = None, [], None
        with torch.cuda.device(self.device):
            try:
                self.base, handle = native.peer_alloc(self.layout["bytes"])
            except RuntimeError as exc:
                handle, error = None, f"rank {self.rank}: {exc}"
            handles = [None] * self.world
            dist.all_gather_object(handles, handle, group=group)
            if error is None and all(h is not None for h in handles):
                try:
                    for r in range(self.world):
                        self.mapped.append(self.base if r == self.rank else native.peer_open(handles[r]))
                except RuntimeError as exc:
                    error = f"rank {self.rank}: {exc}"
            elif error is None:
                error = f"rank {self.rank}: a peer could not allocate its region"
            errors = [None] * self.world
            dist.all_gather_object(errors, error, group=group)
            if any(errors):
                for r, ptr in enumerate(self.mapped):
                    if r != self.rank:
                        native.peer_close(ptr)
                if self.base is not None:
                    native.peer_free(self.base)
                self.base = None
                raise RuntimeError("peer exchange unavailable: " + "; ".join(e for e in errors if e))
        at = lambda name: [b + self.layout[name] for b in self.mapped]      # noqa: E731
        self.recv_ptrs, self.flags_in, self.flags_out = at("recv"), at("flags_in"), at("flags_out")
        self.out_ptrs = (at("out0"), at("out1"))
        self.region = torch.as_tensor(_DeviceSpan(self.base, self.layout["bytes"]), device=self.device)
        lay, rows = self.layout, self.counts[self.rank]
        self.recv = self.region[lay["recv"]:lay["recv"] + lay["recv_bytes"]].view(dtype).view(
            self.first[-1], self.h_local, 3 * head_dim)
        self.out = tuple(
            self.region[lay[n]:lay[n] + rows * heads * head_dim * 2].view(dtype).view(rows, heads, head_dim)
            for n in ("out0", "out1"))
        self.blocks_done = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.epoch, self.inbound = 0, False
        dist.barrier(group=group)                # every region is mapped before anyone stores

    def to_heads(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, producer=None) -> torch.Tensor:
        """``(rows_local, H, D)`` x3 -> ``(S, H/world, 3*D)``: this rank's heads of every row.
        ``producer = (q_weight, k_weight, cos, sin, eps)`` folds the qk-norm + partial rotary step
        into the stores (``native.push_qkv``)."""
        if self.inbound:
            raise RuntimeError("to_heads called twice without to_sequence in between")
        self.epoch += 1
        self.inbound = True
        native.push_qkv(q, k, v, self.recv_ptrs, self.flags_in, self.first, self.rank, self.epoch,
                        self.blocks_done, producer)
        native.wait_flags(self.flags_in[self.rank], self.world, self.epoch, self.limit_ns, self.status,
                          self.device)
        return self.recv

    def to_sequence(self, out_heads: torch.Tensor) -> torch.Tensor:
        """``(S, H/world, D)`` -> ``(rows_local, H, D)``."""
        if not self.inbound:
            raise RuntimeError("to_sequence called without a preceding to_heads")
        self.inbound = False
        slot = self.epoch & 1
        native.push_out(out_heads, self.out_ptrs[slot], self.flags_out, self.first, self.rank, self.epoch,
                        self.blocks_done)
        native.wait_flags(self.flags_out[self.rank], self.world, self.epoch, self.limit_ns, self.status,
                          self.device)
        return self.out[slot]

    def close(self) -> None:
        """Collective: unmaps the peers' regions and frees the own one."""
        if self.base is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)           # nobody stores into a region that is going away
        self.recv = self.out = self.region = None
        with torch.cuda.device(self.device):
            for r, ptr in enumerate(self.mapped):
                if r != self.rank:
                    native.peer_close(ptr)
            dist.barrier(group=self.group)
            native.peer_free(self.base)
        self.base = None


def ulysses_attention(q, k, v, attention_fn, group=None, pack=native.pack_qkv_destination_major,
                      merge=native.merge_heads, pipeline_groups: int = 1,
                      exchange: PeerExchange | None = None, producer=None):
    """Head-shard, run ``attention_fn(q, k, v)`` on ``[1, S, h, D]`` views, shard back.

    ``q, k, v``: ``[1, rows_local, H, D]`` (this rank's rows, every head).  Returns
    ``[1, rows_local, H, D]``.

    The rank's ``H/world`` heads are processed in ``pipeline_groups`` groups.  All input
    exchanges are issued up front as asynchronous collectives, each group's attention waits only
    for its own exchange, and its output exchange runs while the next group computes: apart from
    the first group's input and the last group's output, the all-to-all traffic overlaps the
    attention kernels.  Every rank issues the same collectives in the same order.  The default is
    one group (one exchange each way): measured on 8 B200s two groups lose more to the split
    launches and to the collectives competing with the attention kernel for SMs (9.8 ms against
    8.2 ms per layer) than the overlap wins; on 2 GPUs two groups are 0.5 % faster.

    With ``exchange`` (a ``PeerExchange`` built once for this shape and group) both all-to-alls
    and their pack / merge copies are replaced by stores into the peers' memory; ``producer =
    (q_weight, k_weight, cos, sin, eps)`` then also folds the qk-norm + partial rotary step that
    precedes the exchange into those stores (q and k are passed as the projections wrote them)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if producer is not None and (world == 1 or exchange is None):
        raise ValueError("the producer step is folded into the peer exchange only (world > 1, exchange=...)")
    if world == 1:
        return attention_fn(q, k, v)
    if exchange is not None:
        from .executor import _Stage

        d = q.size(3)
        with _Stage("exchange_to_heads"):
            recv = exchange.to_heads(q[0], k[0], v[0], producer)
        qh, kh, vh = (recv[..., i * d : (i + 1) * d].unsqueeze(0) for i in range(3))
        result = attention_fn(qh, kh, vh)[0].contiguous()
        with _Stage("exchange_to_sequence"):
            return exchange.to_sequence(result).unsqueeze(0)
    rank = dist.get_rank(group)
    rows, heads, d = q.size(1), q.size(2), q.size(3)
    if heads % world:
        raise ValueError(f"heads ({heads}) must divide the Ulysses degree ({world})")
    h_local = heads // world
    counts = row_counts(rows, group)
    total = sum(counts)
    parts = head_groups(h_local, pipeline_groups)

    inbound = []
    for begin, count in parts:
        send = pack(q[0], k[0], v[0], world, begin, count)           # (world, rows, count, 3D)
        inner = count * 3 * d
        recv = torch.empty((total, count, 3 * d), dtype=q.dtype, device=q.device)
        work = dist.all_to_all_single(recv.view(-1), send.view(-1),
                                      output_split_sizes=[c * inner for c in counts],
                                      input_split_sizes=[rows * inner] * world, group=group,
                                      async_op=True)
        inbound.append((work, recv, send))

    out = torch.empty((rows, heads, d), dtype=q.dtype, device=q.device)
    outbound = []
    for (begin, count), (work, recv, send) in zip(parts, inbound):
        work.wait()
        qh, kh, vh = (recv[..., i * d : (i + 1) * d].unsqueeze(0) for i in range(3))
        result = attention_fn(qh, kh, vh)[0].contiguous()            # (S, count, D)
        inner = count * d
        back = torch.empty((world, rows, count, d), dtype=q.dtype, device=q.device)
        work = dist.all_to_all_single(back.view(-1), result.view(-1),
                                      output_split_sizes=[rows * inner] * world,
                                      input_split_sizes=[c * inner for c in counts], group=group,
                                      async_op=True)
        outbound.append((work, back, result, begin))
    for work, back, result, begin in outbound:
        work.wait()
        merge(back, out, begin)
    return out.unsqueeze(0)


def ulysses_anemoi_attention(q, k, v, *, layout: VisualLayout, layer: int,
                             sparse_config: SparseConfig | None = None,
                             quant_config: QuantConfig | None = None,
                             calibration: NVFP4Calibration | None = None, group=None,
                             pipeline_groups: int = 1, exchange: PeerExchange | None = None):
    """``anemoi_attention`` with the heads sharded over the ranks of ``group``."""
    def local(qh, kh, vh):
        return anemoi_attention(qh, kh, vh, layout=layout, layer=layer, sparse_config=sparse_config,
                                quant_config=quant_config, calibration=calibration)
    return ulysses_attention(q, k, v, local, group, pipeline_groups=pipeline_groups, exchange=exchange)


__all__ = ["shard_rows", "row_counts", "reset_row_counts", "head_groups", "exchange_to_heads",
           "exchange_to_sequence", "ulysses_attention", "ulysses_anemoi_attention", "PeerExchange",
           "first_rows", "exchange_region_layout"]
