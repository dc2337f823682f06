"""The host-side stream-ordering checker (``ELF_B200_DEBUG_STREAMS``)."""

import pytest
import torch

from elf_b200.utils import stream_debug as sd


@pytest.fixture(autouse=True)
def _on():
    sd.enable(True)
    yield
    sd.enable(False)


def test_reader_that_waited_passes_and_reader_that_did_not_is_caught():
    buf = torch.zeros(8)
    sd.note_write(buf, "compute", "activation")
    sd.check_read(buf, "compute")  # same stream: program order
    with pytest.raises(sd.StreamOrderError, match="wait_stream / wait_event is missing"):
        sd.check_read(buf, "d2h", "offload copy")
    sd.note_sync("d2h", "compute")
    sd.check_read(buf, "d2h")
    # a later write needs a later wait
    sd.note_write(buf, "compute")
    with pytest.raises(sd.StreamOrderError):
        sd.check_read(buf, "d2h")
    # views share the storage
    sd.note_sync("d2h", "compute")
    sd.check_read(buf[2:4], "d2h")
    # waiting the wrong way round does not help
    other = torch.zeros(4)
    sd.note_write(other, "h2d")
    sd.note_sync("h2d", "compute")
    with pytest.raises(sd.StreamOrderError):
        sd.check_read(other, "compute")


def test_disabled_checker_costs_nothing_and_raises_nothing():
    sd.enable(False)
    buf = torch.zeros(2)
    sd.note_write(buf, "a")
    sd.check_read(buf, "b")
