"""The package's own symmetric-memory runtime (``ELF_B200_SYMM=vmm``): the exchange of file
descriptors between the ranks of a node (CPU, gloo), and - on a GPU - allocation, export,
import and mapping with two processes that share one device (nothing here waits on a kernel of
another process, so one GPU is enough)."""

import os

import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_ranks


def _fd_worker(rank, world):
    from elf_b200.parallel.symm import exchange_fds

    r, w = os.pipe()
    os.write(w, f"from rank {rank}".encode())
    os.close(w)
    theirs = exchange_fds(r, dist.group.WORLD)
    os.close(r)
    assert theirs[rank] == -1
    for peer in range(world):
        if peer == rank:
            continue
        assert theirs[peer] >= 0
        # every peer holds a duplicate of the same pipe end: the first reader gets the text, the rest get b""
        data = os.read(theirs[peer], 64)
        assert data in (b"", f"from rank {peer}".encode()), data
        os.close(theirs[peer])
    dist.barrier()


def test_file_descriptors_cross_between_ranks():
    run_ranks(_fd_worker, 3)


def _vmm_worker(rank, world):
    os.environ["ELF_B200_SYMM"] = "vmm"
    from elf_b200.parallel.symm import SymmetricBuffer

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    n = 1 << 18  # 1 MiB of fp32
    buf = SymmetricBuffer.allocate(n, torch.float32, dist.group.WORLD, dev)
    assert buf.world == world and buf.rank == rank and buf.local.numel() == n and buf.local.dtype == torch.float32
    assert float(buf.local.abs().sum()) == 0.0  # fresh allocations are cleared
    assert buf.addresses[rank] == buf.local.data_ptr() and len(set(buf.addresses)) == world
    buf.local.fill_(float(rank + 1))
    torch.cuda.synchronize()
    dist.barrier()
    arena = buf._handle
    peer = 1 - rank
    theirs = arena.peer_tensor(0)[: 4 * n].view(torch.float32)  # the only peer mapping of a 2-rank group
    assert theirs.data_ptr() == buf.peer_address(peer)
    assert torch.equal(theirs, torch.full_like(theirs, float(peer + 1)))  # a read through the mapping
    dist.barrier()
    theirs[: n // 2].fill_(100.0 + rank)  # a write through the mapping, into the peer's first half
    torch.cuda.synchronize()
    dist.barrier()
    assert torch.equal(buf.local[: n // 2], torch.full((n // 2,), 100.0 + peer, device=dev))
    assert torch.equal(buf.local[n // 2 :], torch.full((n // 2,), float(rank + 1), device=dev))
    dist.barrier()


@pytest.mark.gpu
def test_vmm_arena_maps_a_peer_process_allocation():
    run_ranks(_vmm_worker, 2)
