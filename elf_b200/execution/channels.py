"""Point-to-point channels between pipeline stages.

One ``Channel`` object exists per (producer block, consumer block, direction) and per end.
Traffic on a channel is a FIFO of micro-batch tensors of one fixed shape, so the two ends
always agree on ordering.  Transport:

* NCCL: every channel owns a 2-rank process group (its own communicator and stream), so a
  forward activation and a backward gradient between the same two GPUs never queue behind
  each other — the same reason the reference builds ``group_fwd``/``group_bwd`` per block
  pair (``elf/pipeline.py:640-723``).  Groups are derived from the placement and the
  signatures, which every rank already knows, so no ``all_gather_object`` round is needed
  and each group is created exactly once.
* gloo (CPU): the pipeline group with a per-(channel, micro-batch) tag.
* copy (GPUs of one node, ``ChannelTable.upgrade_to_copy``): after a first step over NCCL has
  told both ends the message size, a channel can switch to a ring of receive slots in the
  consumer's memory (symmetric memory mapped by the producer).  The producer writes a slot with
  the copy engines on a side stream and raises a sequence number; the consumer's compute stream
  waits for it (bounded), copies the slot out and acknowledges it.  No SM-resident kernel
  competes with the persistent GEMMs, which NCCL's send/recv kernels do: next to a
  weight-gradient-sized GEMM a 32 MiB NCCL message in each direction costs the GEMM about as
  long as the message itself takes, the same copy through the copy engines about 5 %
  (``benchmarks/p2p_overlap.py``).

Shape/dtype are learned by the receiving end from a one-off int64 header message that
precedes the first payload (the reference sends 16 floats with a blocking ``recv``,
``elf/execution/block.py:529-570``).  The header is received with ``irecv`` and only waited
for when the consumer actually needs the tensor, so posting a recv early can never block
the host on a peer that has not reached its send yet.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..utils import stream_debug as _sd
from ..utils.metadata import TensorMetadata

__all__ = ["Channel", "ChannelTable", "edge_list"]


def edge_list(signatures) -> List[Tuple[int, int]]:
    """All (producer block, consumer block) pairs, sorted."""
    edges = set()
    for dst, sig in enumerate(signatures):
        for src in sig.get_all_sources():
            if src is not None:
                edges.add((src, dst))
    for src, sig in enumerate(signatures):
        for dst in sig.get_all_targets():
            if dst is not None:
                edges.add((src, dst))
    return sorted(edges)


def _done(work) -> bool:
    try:
        return work.is_completed()
    except Exception:
        return True


class _Pending:
    __slots__ = ("work", "tensor", "mb")

    def __init__(self, mb, work=None, tensor=None):
        self.mb, self.work, self.tensor = mb, work, tensor


class Channel:
    """One end of one directed stream of same-shaped tensors."""

    def __init__(self, src_block: int, dst_block: int, direction: str, peer_global_rank: int, group, device, index: int, n_channels: int):
        self.src_block, self.dst_block, self.direction = src_block, dst_block, direction
        self.peer = peer_global_rank
        self.group = group
        self.device = device
        self.index = index
        self.n_channels = max(1, n_channels)
        self.metadata: Optional[TensorMetadata] = None
        # Only forward channels carry a header: a gradient has the shape of the activation
        # that went the other way, which its receiver produced itself.
        self.header_sent = direction == "bwd"
        self._header_work = None
        self._header_buf: Optional[torch.Tensor] = None
        self._deferred: List[Tuple[int, int]] = []  # (mb, batch) recvs posted before the shape was known
        self._posted: Dict[int, _Pending] = {}
        self._sends: List = []
        # NCCL matches sends and recvs of a communicator purely by order; gloo can use tags.
        # ELF_B200_P2P_STRICT=1 makes gloo behave like NCCL (untagged, one group per channel)
        # so that ordering or size mismatches show up in CPU tests.
        self._tagged = dist.get_backend(group) != "nccl" and os.environ.get("ELF_B200_P2P_STRICT", "0") != "1"
        self.max_message_bytes = 0  # largest payload seen so far (sent or posted), sizes the copy transport's slots
        self.link: Optional["_CopyLink"] = None  # set by switch_to_copy

    def _tag(self, mb: int, header: bool = False) -> int:
        if not self._tagged:
            return 0
        return 1 + ((0 if header else mb + 1) * self.n_channels + self.index)

    # ------------------------------------------------------------------ sending
    def send(self, tensor: torch.Tensor, mb: int) -> None:
        payload = tensor.detach()
        if payload.device != self.device:
            payload = payload.to(self.device)
        payload = payload.contiguous()
        self.max_message_bytes = max(self.max_message_bytes, payload.numel() * payload.element_size())
        if self.link is not None:
            self.link.send(payload)
            return
        if not self.header_sent:
            self.header_sent = True
            head = TensorMetadata(shape=list(payload.shape[1:]), dtype=payload.dtype).to_tensor(self.device)
            self._sends.append((dist.isend(head, dst=self.peer, group=self.group, tag=self._tag(mb, True)), head))
        self._sends.append((dist.isend(payload, dst=self.peer, group=self.group, tag=self._tag(mb)), payload))
        if len(self._sends) > 64:
            self.reap_sends()

    def reap_sends(self, block: bool = False) -> None:
        """Drop handles of completed sends (the handle keeps the payload alive until then)."""
        keep = []
        for work, t in self._sends:
            if block:
                work.wait()
            elif not work.is_completed():
                keep.append((work, t))
        self._sends = keep

    # ------------------------------------------------------------------ receiving
    def set_metadata(self, meta: TensorMetadata) -> None:
        """Tell the receiving end the shape without a header (used for backward channels,
        whose payload has the shape of a tensor this rank produced itself)."""
        self.metadata = meta
        self.header_sent = True

    def post_recv(self, mb: int, batch: int) -> None:
        if self.metadata is None:
            if self._header_work is None and self.direction == "fwd":
                self._header_buf = torch.zeros(TensorMetadata.MAX_SIZE, dtype=torch.int64, device=self.device)
                self._header_work = dist.irecv(self._header_buf, src=self.peer, group=self.group, tag=self._tag(mb, True))
            self._deferred.append((mb, batch))
            return
        self._post(mb, batch)

    def _post(self, mb: int, batch: int) -> None:
        nbytes = batch * self.metadata.dtype.itemsize
        for d in self.metadata.shape:
            nbytes *= d
        self.max_message_bytes = max(self.max_message_bytes, nbytes)
        if self.link is not None:
            self._posted[mb] = _Pending(mb, None, self.link.post((batch, *self.metadata.shape), self.metadata.dtype))
            return
        buf = torch.empty((batch, *self.metadata.shape), dtype=self.metadata.dtype, device=self.device)
        work = dist.irecv(buf, src=self.peer, group=self.group, tag=self._tag(mb))
        self._posted[mb] = _Pending(mb, work, buf)

    def _resolve_header(self) -> None:
        if self.metadata is None:
            if self._header_work is None:
                raise RuntimeError(f"{self}: shape of the incoming tensor is unknown (set_metadata was never called)")
            self._header_work.wait()
            self.metadata = TensorMetadata.from_tensor(self._header_buf.cpu(), device=self.device)
            self._header_work = self._header_buf = None
        for mb, batch in self._deferred:
            self._post(mb, batch)
        self._deferred.clear()

    def wait(self, mb: int) -> torch.Tensor:
        if mb not in self._posted:
            if not any(m == mb for m, _ in self._deferred):
                raise KeyError(f"no recv posted for micro-batch {mb} on channel {self}")
            self._resolve_header()
        pending = self._posted.pop(mb)
        if pending.work is None:  # copy transport: `tensor` holds the ticket of the posted receive
            return self.link.take(pending.tensor)
        pending.work.wait()
        return pending.tensor

    def abandon(self) -> None:
        """Forget posted receives and send handles without waiting for the peer (used when
        a step is given up after an error; the peer may be gone)."""
        self._sends = [(w, t) for w, t in self._sends if not _done(w)]
        if self.link is not None and self._posted:
            # receives that were posted but never taken leave the two ends' sequence numbers
            # out of step: the ring cannot be trusted any more
            self.link.broken = True
        self._posted.clear()
        self._deferred.clear()

    def attach_link(self, link: "_CopyLink") -> None:
        """Route all later traffic of this channel through ``link`` (see ``ChannelTable.upgrade_to_copy``).
        Called between steps, with nothing of this channel in flight."""
        assert not self._posted and not self._deferred, "transport switched with receives in flight"
        self.reap_sends(block=True)
        self.link = link

    def end_step(self) -> None:
        """Forget receives that were posted but not consumed in the step that just ended."""
        if self._posted and self.link is not None:
            self.link.broken = True
        self._posted.clear()

    def reset(self) -> None:
        self.reap_sends(block=True)
        self._posted.clear()
        self._deferred.clear()

    def __repr__(self) -> str:
        return f"Channel({self.src_block}->{self.dst_block} {self.direction}, peer={self.peer})"


class _CopyLink:
    """One end of a channel on the copy transport.

    Every rank of the pipeline holds one symmetric arena.  The consumer's arena has the channel's
    ring (``depth`` slots of ``slot_bytes``) followed by a flag area, the producer's arena a flag
    area; flag 0 of the consumer = sequence number
    of the newest message that has landed, flag 1 of the producer = newest message the consumer
    has copied out (so slot reuse never overtakes the consumer).  Messages are numbered 1, 2, ...
    for the life of the channel and must be taken in the order they were posted, which is the
    order they are sent in (the same rule NCCL imposes)."""

    FLAG_BYTES = 256

    def __init__(self, channel: "Channel", arena: torch.Tensor, peer_arena: torch.Tensor, peer_base_addr: int, at_producer: int, at_consumer: int,
                 slot_bytes: int, depth: int, timeout_ms: float, producer: bool):
        """``arena`` is this rank's symmetric buffer, ``peer_arena`` the peer's as mapped here
        (``peer_base_addr`` its device address).  The channel's region in the consumer's arena
        starts at ``at_consumer`` (``depth`` slots of ``slot_bytes``, then ``FLAG_BYTES`` of flags), its
        region in the producer's arena at ``at_producer`` (``FLAG_BYTES`` of flags)."""
        from ..ops import _ext
        from ..ops import gemm as _gemm

        _ext.require_on_gpu()
        self.ext = _ext.get()
        if not hasattr(self.ext, "p2p_signal"):
            raise RuntimeError("extension built without the p2p flag kernels")
        self.channel = channel
        self.device = channel.device
        self.depth, self.slot_bytes, self.timeout_ms = depth, slot_bytes, timeout_ms
        self.producer = producer
        ring = depth * slot_bytes
        if producer:
            self.buf = None
            self.flags = arena[at_producer : at_producer + self.FLAG_BYTES].view(torch.int32)
            self.peer_buf = peer_arena[at_consumer : at_consumer + ring]
            self.peer_flag_addr = peer_base_addr + at_consumer + ring
        else:
            self.buf = arena[at_consumer : at_consumer + ring]
            self.flags = arena[at_consumer + ring : at_consumer + ring + self.FLAG_BYTES].view(torch.int32)
            self.peer_buf = None
            self.peer_flag_addr = peer_base_addr + at_producer
        self.status = _gemm.status(self.device)
        self.stream = torch.cuda.Stream(self.device)  # producer side: copies run here, behind the compute stream's event
        self.sent = 0  # producer: messages sent
        self.posted = 0  # consumer: receives posted
        self.taken = 0  # consumer: receives taken
        self.where = 100 + channel.index
        self.broken = False

    def _check(self) -> None:
        if self.broken:
            raise RuntimeError(f"{self.channel}: a step was abandoned with receives in flight; the copy transport of this channel is out of step with its peer - rebuild the pipeline")

    # producer ---------------------------------------------------------------------------
    def send(self, payload: torch.Tensor) -> None:
        self._check()
        nbytes = payload.numel() * payload.element_size()
        if nbytes > self.slot_bytes:
            raise RuntimeError(f"{self.channel}: message of {nbytes} bytes exceeds the ring's slot size {self.slot_bytes} (sized from the first step)")
        self.sent += 1
        seq = self.sent
        slot = (seq - 1) % self.depth
        cur = torch.cuda.current_stream(self.device)
        _sd.note_write(payload, cur, "stage output")
        self.stream.wait_stream(cur)  # the payload's producer kernels
        _sd.note_sync(self.stream, cur)
        _sd.check_read(payload, self.stream, "copy into the consumer's ring")
        with torch.cuda.stream(self.stream):
            if seq > self.depth:  # the consumer must have copied out the message this one overwrites
                self.ext.p2p_wait(self.flags, 1, seq - self.depth, self.timeout_ms, self.status, self.where)
            self.peer_buf[slot * self.slot_bytes : slot * self.slot_bytes + nbytes].copy_(payload.reshape(-1).view(torch.uint8), non_blocking=True)
            self.ext.p2p_signal(self.peer_flag_addr, seq)
        payload.record_stream(self.stream)

    # consumer ---------------------------------------------------------------------------
    def post(self, shape, dtype):
        self._check()
        self.posted += 1
        return (self.posted, tuple(shape), dtype)

    def take(self, ticket) -> torch.Tensor:
        self._check()
        seq, shape, dtype = ticket
        if seq != self.taken + 1:
            raise RuntimeError(f"{self.channel}: receives must be consumed in the order they were posted (next is {self.taken + 1}, asked for {seq})")
        self.taken = seq
        slot = (seq - 1) % self.depth
        out = torch.empty(shape, dtype=dtype, device=self.device)
        nbytes = out.numel() * out.element_size()
        self.ext.p2p_wait(self.flags, 0, seq, self.timeout_ms, self.status, self.where)
        out.reshape(-1).view(torch.uint8).copy_(self.buf[slot * self.slot_bytes : slot * self.slot_bytes + nbytes], non_blocking=True)
        self.ext.p2p_signal(self.peer_flag_addr + 4, seq)  # flag 1 of the producer: slot may be reused
        return out


def _arena_layout(sizes: List[int], roles: Dict[int, Tuple[int, int]], world: int, depth: int):
    """Where every channel lives in the ranks' symmetric arenas.  ``sizes[idx]`` is the largest
    message of channel ``idx`` (0: unused so far, the channel stays on NCCL), ``roles[idx]`` its
    ``(producer, consumer)`` ranks.  The consumer's arena holds the channel's ring and the flag
    the producer raises; the producer's arena holds only the flag the consumer raises.  Returns
    ``({idx: (offset in the producer's arena, offset in the consumer's arena, slot bytes)}, arena
    bytes)``; every rank computes the same table (it needs its peers' offsets), and all arenas
    have one size, that of the fullest."""
    cursor = [0] * world
    offsets = {}
    for idx, nbytes in enumerate(sizes):
        if nbytes == 0:
            continue
        producer, consumer = roles[idx]
        slot = (nbytes + 255) // 256 * 256
        offsets[idx] = (cursor[producer], cursor[consumer], slot)
        cursor[consumer] += depth * slot + _CopyLink.FLAG_BYTES
        cursor[producer] += _CopyLink.FLAG_BYTES
    return offsets, max(cursor)


class ChannelTable:
    """All channels touching this rank, keyed by ``(src_block, dst_block, direction, k)``
    where ``src_block`` is the block the *payload* comes from and ``k`` numbers the tensors
    exchanged by that pair of blocks."""

    def __init__(self, placement, signatures, local_rank: int, pp_group, device, *, pp: int, dp: int = 1, dp_rank: int = 0, timeout=None, dedicated_groups: Optional[bool] = None):
        """``placement`` holds pipeline-local ranks; global rank = ``replica * pp + local``.
        With dedicated groups, every process of the job must construct its table at the
        same time (``new_group`` is collective over the world), replicas included."""
        self.channels: Dict[Tuple[int, int, str, int], Channel] = {}
        self._groups = []
        backend = dist.get_backend(pp_group)
        if dedicated_groups is None:
            dedicated_groups = backend == "nccl" or os.environ.get("ELF_B200_P2P_STRICT", "0") == "1"
        # one channel per tensor crossing the edge: a channel carries one fixed shape
        edges = []
        for a, b in edge_list(signatures):
            if placement[a] != placement[b]:
                width = max(1, sum(1 for src in signatures[b].sources if src == a))
                edges += [(a, b, k) for k in range(width)]
        n = 2 * len(edges)
        self.pp_group, self.n_channel_ids, self.device = pp_group, n, device
        self._arena = None
        self._order: List[Tuple[int, int, str, int]] = []  # this rank's channels in creation order (the same relative order on both ends)
        # channel index -> (producer, consumer) as pipeline-local ranks, for every channel of the pipeline
        self._roles: Dict[int, Tuple[int, int]] = {}
        for i, (a, b, k) in enumerate(edges):
            self._roles[2 * i] = (placement[a], placement[b])  # forward: a's output travels to b
            self._roles[2 * i + 1] = (placement[b], placement[a])  # backward: b's input gradient travels to a
        self.transport = "nccl" if backend == "nccl" else backend
        for replica in range(dp if dedicated_groups else 1):
            if not dedicated_groups:
                replica = dp_rank
            offset = replica * pp
            for i, (a, b, k) in enumerate(edges):
                ra, rb = placement[a], placement[b]
                mine = replica == dp_rank and local_rank in (ra, rb)
                for j, direction in enumerate(("fwd", "bwd")):
                    group = pp_group
                    if dedicated_groups:
                        kwargs = {"timeout": timeout} if timeout is not None else {}
                        group = dist.new_group(sorted({offset + ra, offset + rb}), backend=backend, **kwargs)
                        if mine:
                            self._groups.append(group)
                    if not mine:
                        continue
                    src, dst = (a, b) if direction == "fwd" else (b, a)
                    peer_local = rb if local_rank == ra else ra
                    ch = Channel(src, dst, direction, offset + peer_local, group, device, 2 * i + j, n)
                    ch.peer_local = peer_local  # the peer's rank inside the pipeline group
                    ch.is_producer = local_rank == placement[src]
                    self.channels[(src, dst, direction, k)] = ch
                    self._order.append((src, dst, direction, k))

    def get(self, src_block: int, dst_block: int, direction: str, k: int = 0) -> Channel:
        """Channel of the ``k``-th tensor that ``src_block`` sends to ``dst_block``."""
        return self.channels[(src_block, dst_block, direction, k)]

    def upgrade_to_copy(self, depth: int = 4, timeout_ms: float = 60000.0) -> int:
        """Switch every channel that has carried traffic to the copy transport.  Collective over the
        pipeline group (every rank of the job calls it at the same point between two steps):

        1. the ranks gather the largest message every channel has carried;
        2. every rank allocates ONE symmetric arena - the consuming end of a channel holds its ring
           (``depth`` slots) and a flag, the producing end a flag - and the group maps the arenas in
           a single rendezvous.  (One rendezvous per pipeline, entered by all of its ranks: the
           exchange behind it numbers its rounds per process, so ranks that had rendezvoused
           pairwise a different number of times would never meet.)  ``ELF_B200_SYMM=vmm`` takes the
           arena from this package's own runtime instead (``elf_b200.parallel.symm``).
        3. each channel end gets a link onto its region: the consumer's arena holds the ring, the
           producer writes it through its mapping of that arena.

        Returns how many of this rank's channels switched."""
        if self.n_channel_ids == 0:  # nothing crosses ranks (data parallelism only)
            return 0
        if self.transport != "nccl":
            raise RuntimeError("the copy transport needs CUDA tensors and NCCL process groups")
        import torch.distributed._symmetric_memory as symm_mem

        group = self.pp_group
        world = dist.get_world_size(group)
        mine = {ch.index: int(ch.max_message_bytes) for ch in self.channels.values()}
        gathered = [None] * world
        dist.all_gather_object(gathered, mine, group=group)
        sizes = [0] * self.n_channel_ids
        for part in gathered:
            for idx, nbytes in part.items():
                sizes[idx] = max(sizes[idx], nbytes)
        offsets, total = _arena_layout(sizes, self._roles, world, depth)
        if total == 0:
            return 0
        own_runtime = os.environ.get("ELF_B200_SYMM", "torch") == "vmm"
        if own_runtime:
            from ..parallel.symm import SymmetricBuffer

            shared = SymmetricBuffer.allocate(total, torch.uint8, group, self.device)  # cleared, mapped by all, barrier done
            arena, handle = shared.local, shared
        else:
            arena = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            handle = symm_mem.rendezvous(arena, group=group.group_name)
            arena.zero_()
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)  # nobody raises a flag before every arena is zeroed
        self._arena = (arena, handle)
        peers = {}
        switched = 0
        for key in self._order:
            ch = self.channels[key]
            if ch.link is not None or ch.index not in offsets:
                continue
            at_producer, at_consumer, slot = offsets[ch.index]
            if ch.peer_local not in peers:
                if own_runtime:
                    peers[ch.peer_local] = (handle.peer_bytes(ch.peer_local), handle.peer_address(ch.peer_local))
                else:
                    peers[ch.peer_local] = (handle.get_buffer(ch.peer_local, (total,), torch.uint8), int(handle.buffer_ptrs[ch.peer_local]))
            peer_arena, peer_addr = peers[ch.peer_local]
            ch.attach_link(_CopyLink(ch, arena, peer_arena, peer_addr, at_producer, at_consumer, slot, depth, timeout_ms, ch.is_producer))
            switched += 1
        self.transport = "copy"
        return switched

    def reset(self) -> None:
        for ch in self.channels.values():
            ch.reset()

    def destroy(self) -> None:
        for g in self._groups:
            try:
                dist.destroy_process_group(g)
            except Exception:
                pass
        self._groups.clear()
