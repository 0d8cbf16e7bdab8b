"""Batch-sharded data-parallel inference on the GPUs of one node.

Every op of the path is independent across batch rows, so each rank (one process per GPU) runs the whole network on its own
slice of the batch with replicated weights; the only exchange is the all-gather of the fp32 logits at the end.  Nothing
else crosses NVLink, and no kernel of this package reads another GPU's memory.  The reference has no multi-GPU inference
at all (its only collective use is ChainerMN in a training example).
"""
import os

import numpy as np
import torch
import torch.distributed as dist


def env_world():
    """(rank, local_rank, world_size) from the torchrun environment; (0, 0, 1) when launched plainly."""
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def init(backend=None):
    rank, local_rank, world = env_world()
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, local_rank, world


def shard_bounds(total, world, rank):
    """Contiguous slice [begin, end) of `total` batch rows owned by `rank`; the first total % world ranks hold one extra row."""
    base, extra = divmod(int(total), int(world))
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def gather_logits(local_logits, world, out=None):
    """All-gather of equally sized [n_local, classes] fp32 blocks -> [n_local * world, classes] on every rank."""
    if world == 1:
        return local_logits
    if out is None:
        out = torch.empty((local_logits.shape[0] * world,) + tuple(local_logits.shape[1:]), dtype=local_logits.dtype, device=local_logits.device)
    dist.all_gather_into_tensor(out, local_logits.contiguous())
    return out


def gather_ragged(local_rows, total, world, rank):
    """All-gather for a batch that does not divide evenly: pads every shard to the largest, gathers, drops the padding."""
    if world == 1:
        return local_rows
    per = (total + world - 1) // world
    pad = torch.zeros((per,) + tuple(local_rows.shape[1:]), dtype=local_rows.dtype, device=local_rows.device)
    pad[: local_rows.shape[0]] = local_rows
    full = gather_logits(pad, world)
    parts = []
    for r in range(world):
        b, e = shard_bounds(total, world, r)
        parts.append(full[r * per: r * per + (e - b)])
    return torch.cat(parts, dim=0)


def max_over_ranks(value, device, world):
    """Max of a Python float over all ranks (the timing rule for multi-GPU numbers)."""
    if world == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sharded_matmul_integer(a_local, b, a_zero_point=None, b_zero_point=None, total_rows=None, world=1, rank=0, gather=True, matmul=None):
    """MatMulInteger (runtime/ops/quantize.cc:96-114) with the rows of A sharded over the ranks and B replicated: every output row
    depends on one row of A only, so each rank computes Y[begin:end] = (A[begin:end] - za) . (B - zb) for its slice
    shard_bounds(total_rows, world, rank) with no exchange, and the optional all-gather of the int32 rows is the only traffic.
    a_local: this rank's rows; total_rows: rows of the whole A (default: a_local's, i.e. one rank).  matmul: the single-GPU op
    (default ops.MatMulInteger; the CPU-rank tests pass a stand-in).  Returns the whole Y on every rank (gather=True) or this
    rank's rows."""
    if matmul is None:
        from . import ops
        matmul = ops.MatMulInteger
    total_rows = a_local.shape[0] if total_rows is None else int(total_rows)
    begin, end = shard_bounds(total_rows, world, rank)
    if a_local.shape[0] != end - begin:
        raise ValueError("rank %d holds %d rows of A, its shard of %d rows over %d ranks is [%d, %d)" % (rank, a_local.shape[0], total_rows, world, begin, end))
    y_local = matmul(a_local, b, a_zero_point, b_zero_point)
    if not gather or world == 1:
        return y_local
    return gather_ragged(y_local, total_rows, world, rank)


def gpu_numa_cpus(device_index):
    """CPUs of the NUMA node the GPU hangs off (from sysfs), or None when the machine has one node or the answer is unknown."""
    try:
        bus = torch.cuda.get_device_properties(device_index).pci_bus_id
        dom = torch.cuda.get_device_properties(device_index).pci_domain_id
        dev = torch.cuda.get_device_properties(device_index).pci_device_id
        path = "/sys/bus/pci/devices/%04x:%02x:%02x.0/numa_node" % (dom, bus, dev)
        node = int(open(path).read().strip())
        if node < 0 or not os.path.isdir("/sys/devices/system/node/node1"):
            return None
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        return cpus or None
    except Exception:
        return None


def pinned_like(shape, dtype, device_index):
    """Pinned host buffer whose pages are first touched from a CPU of the GPU's NUMA node (first-touch placement), so that the
    copies do not cross the socket interconnect on a two-socket host.  On a one-node host this is a plain pinned allocation."""
    cpus = gpu_numa_cpus(device_index) if torch.cuda.is_available() else None
    old = None
    if cpus:
        try:
            old = os.sched_getaffinity(0)
            os.sched_setaffinity(0, cpus & old or old)
        except OSError:
            old = None
    try:
        t = torch.zeros(shape, dtype=dtype).pin_memory()
    finally:
        if old is not None:
            os.sched_setaffinity(0, old)
    return t


class InferenceEngine:
    """One rank's share of a data-parallel inference job: a calibrated network captured in two CUDA graphs (two input slots,
    two logits buffers) used alternately, a communication stream on which the logits all-gather of step i runs while step
    i + 1 computes, and pinned host buffers for the results.

    Results: every rank holds the logits of the whole job on the device after a step (all-gather).  The host copy is
    what the rank needs: rank 0 receives the whole job's logits, the other ranks their own rows."""

    def __init__(self, net, world=1, fold=False, rank=0, input_dtype=torch.float32):
        """input_dtype: torch.float32 -- the network's own input, quantized on the device by the stem's fused QuantizeLinear -- or
        torch.uint8 -- batches the host has already quantized with the network's input scale (QuantizeLinear(x, net.in_scale, 0));
        the results are the same bytes, a quarter of the bytes cross PCIe."""
        self.net, self.world, self.fold, self.rank = net, world, fold, rank
        assert input_dtype in (torch.float32, torch.uint8)
        self.input_dtype = input_dtype
        dev = net.device
        self.x_dev = torch.empty((net.batch, 3, net.image, net.image), dtype=input_dtype, device=dev)
        self.graph = None
        self.logits = None
        self.all_logits = None
        self.host_logits = None
        self.slots = None
        self._flip = 0

    def prepare(self, calib_x):
        """Calibrates on calib_x and captures the two graphs.  The device-resident input of step_device is self.x_dev (call
        set_resident_input after changing it)."""
        if self.input_dtype == torch.float32:
            self.x_dev.copy_(calib_x)
            self.net.calibrate(self.x_dev)
        else:
            from . import ops
            calib_dev = calib_x.to(self.net.device)
            if not self.net.calibrated:
                self.net.calibrate(calib_dev)
            self.x_dev.copy_(ops.QuantizeLinear(calib_dev, self.net.in_scale, np.uint8(0)))
            del calib_dev
        dev = self.net.device
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        self.comm_stream = torch.cuda.Stream(dev)
        self.h2d_stream, self.d2h_stream = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.slots = []
        for k in range(2):
            x = self.x_dev if k == 0 else torch.empty_like(self.x_dev)
            if k:
                x.copy_(self.x_dev)
            graph, logits = self.net.capture(x, fold=self.fold)
            n, c = logits.shape
            rows = n * self.world if (self.world > 1 and self.rank == 0) else n
            self.slots.append({
                "x": x, "graph": graph, "logits": logits,
                "all": torch.empty((n * self.world, c), dtype=torch.float32, device=dev) if self.world > 1 else logits,
                "host": pinned_like((rows, c), torch.float32, idx),
                "in_ready": torch.cuda.Event(), "in_free": torch.cuda.Event(), "out_ready": torch.cuda.Event(),
                "gathered": torch.cuda.Event(), "host_ready": torch.cuda.Event(), "busy": False})
        s0 = self.slots[0]
        self.graph, self.logits, self.all_logits, self.host_logits = s0["graph"], s0["logits"], s0["all"], s0["host"]

    def set_resident_input(self, x):
        """Makes x (device or pinned host, NCHW, the engine's input dtype) the input of both slots for step_device."""
        for s in self.slots:
            s["x"].copy_(x)

    def _gather_async(self, s, compute):
        """All-gather of slot s's logits on the communication stream, ordered after the slot's graph on `compute`."""
        s["out_ready"].record(compute)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(s["out_ready"])
            gather_logits(s["logits"], self.world, s["all"])
            s["gathered"].record(self.comm_stream)

    def step_device(self):
        """One pass over the resident batch; returns the device tensor that will hold the whole job's logits once the
        communication stream has caught up (drain() orders the current stream after that).  The two slots alternate, so the
        all-gather of one step overlaps the next step's kernels instead of sitting between two graph replays."""
        compute = torch.cuda.current_stream()
        s = self.slots[self._flip]
        self._flip ^= 1
        if self.world > 1:
            compute.wait_event(s["gathered"])  # the gather that read this slot's logits two steps ago
        s["graph"].replay()
        if self.world > 1:
            self._gather_async(s, compute)
        return s["all"]

    def drain(self):
        """Orders the current stream after every all-gather issued so far (call before recording the end of a timed region)."""
        if self.world > 1:
            compute = torch.cuda.current_stream()
            for s in self.slots:
                compute.wait_event(s["gathered"])

    def _result_view(self, s):
        """What this rank copies to the host: rank 0 the whole job's logits, the others their own rows."""
        return s["all"] if (self.world > 1 and self.rank == 0) else s["logits"]

    def run_host(self, x_host_pinned):
        """Public end-to-end call: pinned host NCHW batch (the engine's input dtype) in, host logits out (rank 0: the whole job's;
        others: own rows)."""
        s = self.slots[0]
        compute = torch.cuda.current_stream()
        s["x"].copy_(x_host_pinned, non_blocking=True)
        s["graph"].replay()
        if self.world > 1:
            self._gather_async(s, compute)
            compute.wait_event(s["gathered"])
        s["host"].copy_(self._result_view(s), non_blocking=True)
        compute.synchronize()
        return s["host"]

    # ---- pipelined end-to-end call ------------------------------------------------------------------------------------
    def run_stream(self, batches):
        """Public streaming call: an iterable of pinned host NCHW batches (the engine's input dtype) in, one host logits array out per batch, in
        order (rank 0: the whole job's rows; other ranks: their own).  Batch i+1 crosses PCIe while batch i computes and batch
        i-1's logits are gathered and copied back.  The returned array of batch i is valid until batch i+2 is submitted."""
        compute = torch.cuda.current_stream()
        pending = []
        for i, xb in enumerate(batches):
            s = self.slots[i % 2]
            if s["busy"]:  # hand out this slot's previous result (its copy-out has then finished) before the slot is reused
                yield self._finish(pending.pop(0))
            with torch.cuda.stream(self.h2d_stream):
                self.h2d_stream.wait_event(s["in_free"])
                s["x"].copy_(xb, non_blocking=True)
                s["in_ready"].record(self.h2d_stream)
            compute.wait_event(s["in_ready"])
            s["graph"].replay()
            s["in_free"].record(compute)
            if self.world > 1:
                self._gather_async(s, compute)
                last = s["gathered"]
            else:
                s["out_ready"].record(compute)
                last = s["out_ready"]
            with torch.cuda.stream(self.d2h_stream):
                self.d2h_stream.wait_event(last)
                s["host"].copy_(self._result_view(s), non_blocking=True)
                s["host_ready"].record(self.d2h_stream)
            s["busy"] = True
            pending.append(s)
        while pending:
            yield self._finish(pending.pop(0))

    @staticmethod
    def _finish(s):
        s["host_ready"].synchronize()
        s["busy"] = False
        return s["host"]
