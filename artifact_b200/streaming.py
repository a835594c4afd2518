"""Aggregation with host-resident inputs and outputs.

Upstream keeps features on the host until each training run moves them to the GPU
(ROF_evaluation/ROF_main.py:133-161) and every call of its extension works on device tensors.
A caller that streams feature matrices from host memory pays a host->device copy before and a
device->host copy after every pass; `HostStreamedAggregator` hides both behind the aggregation:
inputs and outputs are double-buffered on the device, uploads run on their own stream, downloads
on another, so the upload of pass k+1 and the download of pass k-1 overlap the kernels of pass k.
A pass is then bounded by max(copy, aggregate) instead of their sum.
"""
import contextlib
import os

import torch


def _cpulist(text):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        a, _, b = part.partition("-")
        cpus.update(range(int(a), int(b or a) + 1))
    return cpus


def device_host_node(device_index, sysfs="/sys"):
    """(numa node, cpus of that node) of the host socket the GPU's PCIe link hangs off, or (None, set())
    where the platform does not say (one node, a VM that hides the topology, no sysfs)."""
    try:
        p = torch.cuda.get_device_properties(device_index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        node = int(open(f"{sysfs}/bus/pci/devices/{bdf}/numa_node").read())
        if node < 0:
            return None, set()
        return node, _cpulist(open(f"{sysfs}/devices/system/node/node{node}/cpulist").read())
    except Exception:
        return None, set()


@contextlib.contextmanager
def near_device(device_index, sysfs="/sys"):
    """Run the body on cores of the GPU's own host socket, so that pinned buffers allocated (and first
    touched) inside it are local to the GPU's PCIe root: a copy between a GPU and memory of the other
    socket crosses the inter-socket link, which all GPUs of a box then share.  Yields the node or None;
    the thread's affinity is put back afterwards (compute threads started later see all cores again)."""
    node, cpus = device_host_node(device_index, sysfs)
    old = None
    try:
        if node is not None and hasattr(os, "sched_getaffinity"):
            mine = os.sched_getaffinity(0)
            if cpus & mine and (cpus & mine) != mine:
                old = mine
                os.sched_setaffinity(0, cpus & mine)
            elif not (cpus & mine):
                node = None
        yield node
    finally:
        if old is not None:
            os.sched_setaffinity(0, old)


def pinned_near(device_index, shape, dtype=torch.float32):
    """a pinned host tensor placed on the GPU's host socket where that can be told (near_device)"""
    with near_device(device_index):
        t = torch.empty(shape, dtype=dtype, pin_memory=True)
        t.zero_()                      # first touch inside the binding
    return t


class _Slot:
    def __init__(self, x_dev, out_dev, run):
        self.x_dev, self.out_dev, self.run = x_dev, out_dev, run
        self.uploaded = torch.cuda.Event()
        self.computed = torch.cuda.Event()
        self.downloaded = torch.cuda.Event()
        self.used = False


class HostStreamedAggregator:
    """submit(h_x, h_out): h_out = aggregate(h_x) for pinned host tensors, asynchronously.

    slots: list of (x_dev, out_dev, run) — `x_dev` the device tensor an upload lands in (this
    rank's rows of the feature matrix), `out_dev` the device tensor the pass writes, `run()` the
    call that enqueues the pass on the current stream (for example
    ``lambda: plan.aggregate(x_full, degrees, mode, out=out_dev, tiles=tiles)`` or a
    PipelinedAggregator's aggregate).  Two slots give double buffering.
    """

    def __init__(self, slots, device):
        self.device = torch.device(device)
        self.slots = [_Slot(*s) for s in slots]
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.seq = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def submit(self, h_x, h_out, aggregate=True):
        """Enqueue upload -> pass -> download for one pair of pinned host buffers.  With
        aggregate=False only the two copies run (the copy-only time of the same schedule)."""
        if not (h_x.is_pinned() and h_out.is_pinned()):
            raise RuntimeError("host buffers must be pinned (torch.empty(..., pin_memory=True))")
        s = self.slots[self.seq % len(self.slots)]
        self.seq += 1
        cur = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self.s_in):
            if s.used:
                self.s_in.wait_event(s.computed)          # the slot's previous pass has read its input
            s.x_dev.copy_(h_x, non_blocking=True)
            s.uploaded.record(self.s_in)
        cur.wait_event(s.uploaded)
        if s.used:
            cur.wait_event(s.downloaded)                  # the slot's previous result is on the host
        if aggregate:
            s.run()
        s.computed.record(cur)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(s.computed)
            h_out.copy_(s.out_dev, non_blocking=True)
            s.downloaded.record(self.s_out)
        s.used = True
        self.h2d_bytes += h_x.numel() * h_x.element_size()
        self.d2h_bytes += h_out.numel() * h_out.element_size()
        return s

    def join(self):
        """Make the current stream wait until every submitted result is in host memory."""
        cur = torch.cuda.current_stream(self.device)
        for s in self.slots:
            if s.used:
                cur.wait_event(s.downloaded)

    def synchronize(self):
        for s in self.slots:
            if s.used:
                s.downloaded.synchronize()
