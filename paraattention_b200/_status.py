"""Device status words and their host mirrors.

Every bounded wait in the kernels reports a timeout by writing a ``pa_device_status`` code into a
device word and makes every later launch that is given the same word return at its entry, so a
stuck exchange can never hang a GPU - but it also means that from then on results are garbage
until somebody looks at the word. ``StatusMirror`` makes the host look without adding a device
synchronisation to the call path: after each launch the word is copied (asynchronously, 4 bytes)
into pinned host memory, and before each launch the host copy - which by then holds the state
after some earlier launch - is read. A timeout therefore surfaces as a ``PaError(PA_ETIMEDOUT)``
on one of the next calls (at the latest after the next synchronisation), where the reference's
NCCL path would raise or abort on a stuck collective. ``reset()`` clears both words.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import _lib as L


class StatusMirror:
    def __init__(self, word: torch.Tensor):
        assert word.dtype == torch.int32 and word.numel() == 1
        self.word = word
        host = torch.zeros(1, dtype=torch.int32)
        # (pinning needs a CUDA runtime; a CPU word - the unit tests - gets a plain host copy)
        self.host = host.pin_memory() if word.device.type == "cuda" else host

    def check(self) -> None:
        """Raise if an earlier launch reported a timed-out wait. Reads host memory only."""
        code = int(self.host[0])
        if code != 0:
            raise L.PaError(L.PA_ETIMEDOUT,
                            L.DEV_STATUS_NAMES.get(code, f"device status {code}") +
                            " (the status word is sticky: call reset() once the cause is dealt with)")

    def refresh(self) -> None:
        """Queue a copy of the device word to the host mirror on the current stream."""
        self.host.copy_(self.word, non_blocking=True)

    def check_now(self) -> None:
        """Synchronising form: read the device word itself."""
        self.host.copy_(self.word)
        self.check()

    def reset(self) -> None:
        self.word.zero_()
        self.host.zero_()


_single: Dict[int, StatusMirror] = {}


def single_gpu_status(device: torch.device) -> StatusMirror:
    """The status word the single-GPU attention ops of this process share on ``device``."""
    m = _single.get(device.index)
    if m is None:
        m = StatusMirror(torch.zeros(1, dtype=torch.int32, device=device))
        _single[device.index] = m
    return m


def all_mirrors():
    return list(_single.values())
