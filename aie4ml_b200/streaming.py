"""Host-to-host execution of a lowered model as a three-stage stream pipeline.

A lowered graph is independent along its leading (batch) axis, so a host batch of any length is
cut into chunks of the plan's own batch size and the chunks flow through

    copy-in stream   : pinned host rows  -> device input buffers of slot s
    compute stream   : the plan's launches (or its captured CUDA graph) on slot s
    copy-out stream  : device output buffers of slot s -> pinned host rows

with ``depth`` slots in flight, ordered by CUDA events only (no host synchronisation inside the
loop).  Copy-in of chunk i+1, compute of chunk i and copy-out of chunk i-1 overlap, so the step
costs max(H2D, compute, D2H) instead of their sum; on a PCIe-attached GPU the two copy directions
run concurrently.  This is the executor behind ``CudaModel.predict`` when ``Iterations`` > 1
(the reference runs its simulator once per iteration, ``src/aie4ml/simulation.py:199-245``).

Slots share one set of device constants; each slot owns its activation buffers.
"""

from __future__ import annotations

from typing import Dict, List, Optional

from . import lib as _lib
from .runtime import Plan


def gpu_local_cpus(device_index: int) -> Optional[List[int]]:
    """CPUs on the NUMA node nearest to a CUDA device (NVML's ideal affinity, read-only query), restricted to the
    CPUs this process may use; None when NVML or the query is unavailable."""
    import os

    try:
        import pynvml
        import torch

        props = torch.cuda.get_device_properties(device_index)
        bus = f'{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0'
        pynvml.nvmlInit()
        try:
            handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            n_cpu = os.cpu_count() or 1
            words = pynvml.nvmlDeviceGetCpuAffinity(handle, (n_cpu + 63) // 64)
        finally:
            pynvml.nvmlShutdown()
        cpus = [w * 64 + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1]
        allowed = os.sched_getaffinity(0) if hasattr(os, 'sched_getaffinity') else set(range(n_cpu))
        cpus = [c for c in cpus if c in allowed]
        return cpus or None
    except Exception:
        return None


def gpu_numa_node(device_index: int) -> Optional[int]:
    """NUMA node the GPU's PCIe slot hangs off (sysfs), or None when the platform does not say."""
    try:
        import torch

        props = torch.cuda.get_device_properties(device_index)
        bdf = f'{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0'
        with open(f'/sys/bus/pci/devices/{bdf}/numa_node') as fh:
            node = int(fh.read().strip())
        return node if node >= 0 else None
    except Exception:
        return None


_SYS_SET_MEMPOLICY = 238      # x86-64
_MPOL_DEFAULT, _MPOL_PREFERRED = 0, 1


def _set_mempolicy(mode: int, node: Optional[int]) -> bool:
    """set_mempolicy(2) for the calling thread through the raw system call (no libnuma here).  False when the
    kernel refuses (another architecture, a cpuset without that node, a sandbox)."""
    import ctypes
    import platform

    if platform.machine() != 'x86_64':
        return False
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        if node is None:
            return libc.syscall(_SYS_SET_MEMPOLICY, mode, None, 0) == 0
        mask = (ctypes.c_ulong * 16)()
        mask[node // 64] = 1 << (node % 64)
        return libc.syscall(_SYS_SET_MEMPOLICY, mode, mask, 16 * 64 + 1) == 0
    except Exception:
        return False


class near_gpu:
    """Context manager: host buffers allocated and pinned inside the block land in the memory of the NUMA node the
    GPU is attached to, so copies between them and the GPU do not cross the socket interconnect.  Two means, both
    undone on exit: the calling thread prefers that node's memory (set_mempolicy, which works even when this
    process may not run on that node's CPUs), and it runs on the node's CPUs where it is allowed to (first
    touch).  A no-op when the topology cannot be read."""

    def __init__(self, device_index: int):
        self.cpus = gpu_local_cpus(device_index)
        self.node = gpu_numa_node(device_index)
        self.saved = None
        self.policy_set = False

    def __enter__(self):
        import os

        if self.node is not None:
            self.policy_set = _set_mempolicy(_MPOL_PREFERRED, self.node)
        if self.cpus and hasattr(os, 'sched_setaffinity'):
            self.saved = os.sched_getaffinity(0)
            os.sched_setaffinity(0, self.cpus)
        return self

    def __exit__(self, *exc):
        import os

        if self.saved is not None:
            os.sched_setaffinity(0, self.saved)
        if self.policy_set:
            _set_mempolicy(_MPOL_DEFAULT, None)
        return False

    def describe(self) -> dict:
        return {'requested': True, 'gpu_numa_node': self.node, 'memory_policy_preferred_node': bool(self.policy_set),
                'ran_on_node_cpus': len(self.cpus) if self.cpus else 0}


class HostPipeline:
    def __init__(self, ctx, depth: int = 3, *, first_plan: Optional[Plan] = None, fuse_rowop_add: bool = True,
                 dense_algo: int = _lib.ALGO_AUTO, use_graph: bool = True):
        """``first_plan``: an existing plan of ``ctx`` to use as slot 0 (its fusion and algorithm
        settings apply to every slot); otherwise ``fuse_rowop_add`` / ``dense_algo`` configure a new one."""
        import torch

        if depth < 1:
            raise ValueError('depth must be at least 1')
        self.torch = torch
        first = first_plan or Plan(ctx, fuse_rowop_add=fuse_rowop_add, dense_algo=dense_algo)
        self.plans: List[Plan] = [first]
        for _ in range(depth - 1):
            self.plans.append(Plan(ctx, device=str(first.device), fuse_rowop_add=first.fuse_rowop_add,
                                   fuse_attention=first.fuse_attention, merge_attention_heads=first.merge_attention_heads,
                                   merge_parallel_dense=first.merge_parallel_dense,
                                   fuse_dense_chain=first.fuse_dense_chain,
                                   dense_algo=first.dense_algo,
                                   share_params=first))
        self.device = first.device
        graph = first.graph
        self.in_names = list(graph.input_tensor_names)
        self.out_names = list(graph.output_tensor_names)
        self.chunk_rows = int(graph.tensors[self.in_names[0]].shape[0])
        for n in self.in_names + self.out_names:
            if int(graph.tensors[n].shape[0]) != self.chunk_rows:
                raise ValueError(f'{n}: leading extent differs from the batch size {self.chunk_rows}; '
                                 'the graph cannot be streamed along its first axis.')
        if use_graph:
            for p in self.plans:
                if p.graph_exec is None:
                    p.capture()
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        mk = lambda: [torch.cuda.Event() for _ in self.plans]
        self.ev_in, self.ev_run, self.ev_out = mk(), mk(), mk()
        self.launches_per_chunk = len(first.launches)

    def chunks_for(self, rows: int) -> int:
        return (int(rows) + self.chunk_rows - 1) // self.chunk_rows

    def run(self, host_in: Dict[str, 'object'], host_out: Dict[str, 'object'], launches: bool = True) -> int:
        """Stream ``host_in[name][r]`` for every row r through the model into ``host_out``.

        Host tensors are torch CPU tensors (pinned for asynchronous copies) shaped ``[rows, ...]``
        with the graph tensor's trailing extents; ``rows`` need not be a multiple of the chunk.  A
        short last chunk runs at full chunk size over whatever the slot's buffers hold beyond the
        copied rows (operators never mix rows), and only its valid rows are copied back.
        ``launches=False`` leaves the kernels out and keeps every copy and every event: what the host's memory and
        the PCIe link allow for this chunking (a measurement aid).
        Returns the number of chunks.  The call only enqueues: the caller's current stream is made to
        wait for all three pipeline streams, so synchronise it (or use ``run_and_wait``) before
        reading ``host_out``.
        """
        torch = self.torch
        rows = int(host_in[self.in_names[0]].shape[0])
        for n in self.in_names:
            if int(host_in[n].shape[0]) != rows:
                raise ValueError(f'{n}: every input needs the same number of rows ({rows}).')
        for n in self.out_names:
            if int(host_out[n].shape[0]) != rows:
                raise ValueError(f'{n}: output buffer needs {rows} rows.')
        n_chunks = self.chunks_for(rows)
        depth = len(self.plans)
        origin = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(origin)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(start)
        for c in range(n_chunks):
            slot = c % depth
            plan = self.plans[slot]
            r0 = c * self.chunk_rows
            r1 = min(rows, r0 + self.chunk_rows)
            with torch.cuda.stream(self.s_in):
                if c >= depth:
                    self.s_in.wait_event(self.ev_run[slot])     # the slot's inputs have been consumed
                for n in self.in_names:
                    plan.tensor_of(n)[: r1 - r0].copy_(host_in[n][r0:r1], non_blocking=True)
                self.ev_in[slot].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[slot])
                if c >= depth:
                    self.s_run.wait_event(self.ev_out[slot])    # the slot's outputs have been read back
                if launches:
                    plan.run()
                self.ev_run[slot].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[slot])
                for n in self.out_names:
                    host_out[n][r0:r1].copy_(plan.tensor_of(n)[: r1 - r0], non_blocking=True)
                self.ev_out[slot].record(self.s_out)
        for s in (self.s_in, self.s_run, self.s_out):
            origin.wait_stream(s)
        return n_chunks

    def run_and_wait(self, host_in, host_out) -> int:
        n = self.run(host_in, host_out)
        self.torch.cuda.synchronize(self.device)
        self.plans[0].check_status()
        return n
