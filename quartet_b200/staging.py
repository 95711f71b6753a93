"""Host -> device staging for the layer's inputs: pinned host tensors are copied into resident device
buffers on a side stream, one item ahead of the compute stream, so that the PCIe transfer of the
next layer's activations and output-gradients runs under the current layer's kernels.

The reference keeps its batches on the device through torch's DataLoader + `.to(device,
non_blocking=True)` (src/data/utils.py, src/optim/base.py:170-200 in the reference tree); this is the
same idea restated for the per-layer inputs of the quantized-linear path.
"""
from __future__ import annotations

from typing import Dict, Hashable, Sequence

import torch


class HostStager:
    """One resident device buffer per key; `prefetch` enqueues the copies on the side stream after
    the compute stream's last recorded use of that buffer, `acquire` makes the compute stream wait
    for them and returns the device tensors, `release` records that the compute stream is done."""

    def __init__(self, device: torch.device):
        if torch.device(device).type != "cuda":
            raise RuntimeError("HostStager stages into CUDA memory; there is no CPU path")
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(device=self.device)
        self._bufs: Dict[Hashable, Sequence[torch.Tensor]] = {}
        self._ready: Dict[Hashable, torch.cuda.Event] = {}
        self._free: Dict[Hashable, torch.cuda.Event] = {}
        self.bytes_copied = 0

    def register(self, key: Hashable, device_tensors: Sequence[torch.Tensor]) -> None:
        self._bufs[key] = tuple(device_tensors)

    def prefetch(self, key: Hashable, host_tensors: Sequence[torch.Tensor]) -> None:
        bufs = self._bufs[key]
        if len(bufs) != len(host_tensors):
            raise ValueError("one host tensor per registered device buffer")
        for h in host_tensors:
            if not h.is_pinned():
                raise ValueError("host tensors must be pinned for the copy to be asynchronous")
        free = self._free.pop(key, None)
        if free is not None:
            self.stream.wait_event(free)
        with torch.cuda.stream(self.stream):
            for d, h in zip(bufs, host_tensors):
                d.detach().copy_(h, non_blocking=True)
                self.bytes_copied += h.numel() * h.element_size()
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self._ready[key] = ev

    def acquire(self, key: Hashable) -> Sequence[torch.Tensor]:
        ev = self._ready.pop(key, None)
        if ev is None:
            raise RuntimeError(f"nothing was prefetched for {key!r}")
        torch.cuda.current_stream(self.device).wait_event(ev)
        return self._bufs[key]

    def release(self, key: Hashable) -> None:
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._free[key] = ev


class HostDrain:
    """Device -> pinned host copies of a step's results on their own stream, so that they leave over PCIe
    while the compute stream runs the next layer.  `push` orders the copy after everything the compute
    stream has been given so far; `join` makes the compute stream wait for all copies pushed so far."""

    def __init__(self, device: torch.device):
        if torch.device(device).type != "cuda":
            raise RuntimeError("HostDrain copies out of CUDA memory; there is no CPU path")
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(device=self.device)
        self.bytes_copied = 0

    def push(self, host_tensor: torch.Tensor, device_tensor: torch.Tensor) -> None:
        if not host_tensor.is_pinned():
            raise ValueError("the host tensor must be pinned for the copy to be asynchronous")
        if host_tensor.shape != device_tensor.shape or host_tensor.dtype != device_tensor.dtype:
            raise ValueError(f"host buffer {tuple(host_tensor.shape)} {host_tensor.dtype} does not match the result "
                             f"{tuple(device_tensor.shape)} {device_tensor.dtype}")
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            host_tensor.copy_(device_tensor, non_blocking=True)
        device_tensor.record_stream(self.stream)
        self.bytes_copied += host_tensor.numel() * host_tensor.element_size()

    def join(self) -> None:
        torch.cuda.current_stream(self.device).wait_stream(self.stream)
