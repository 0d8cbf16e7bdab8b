"""Batch-sharded data-parallel inference on the GPUs of one node.

Every op of the path is independent across batch rows, so each rank (one process per GPU) runs the whole network on its own
slice of the batch with replicated weights; the only exchange is the all-gather of the fp32 logits at the end.  Nothing
else crosses NVLink, and no kernel of this package reads another GPU's memory.  The reference has no multi-GPU inference
at all (its only collective use is ChainerMN in a training example).
"""
import os

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


class InferenceEngine:
    """One rank's share of a data-parallel inference job: a calibrated network captured in a CUDA graph, a pinned host
    staging buffer for inputs and one for the gathered logits."""

    def __init__(self, net, world=1, fold=False):
        self.net, self.world, self.fold = net, world, fold
        dev = net.device
        self.x_dev = torch.empty((net.batch, 3, net.image, net.image), dtype=torch.float32, device=dev)
        self.graph = None
        self.logits = None
        self.all_logits = None
        self.host_logits = None
        self.slots = None

    def prepare(self, calib_x):
        self.x_dev.copy_(calib_x)
        self.net.calibrate(self.x_dev)
        self.graph, self.logits = self.net.capture(self.x_dev, fold=self.fold)
        n, c = self.logits.shape
        self.all_logits = torch.empty((n * self.world, c), dtype=torch.float32, device=self.net.device)
        self.host_logits = torch.empty((n * self.world, c), dtype=torch.float32).pin_memory()

    def step_device(self):
        """One pass over the batch already resident in self.x_dev; logits of every rank end up in self.all_logits."""
        self.graph.replay()
        if self.world > 1:
            gather_logits(self.logits, self.world, self.all_logits)
            return self.all_logits
        return self.logits

    def run_host(self, x_host_pinned):
        """Public end-to-end call: pinned host fp32 NCHW batch in, host logits of the whole job out."""
        self.x_dev.copy_(x_host_pinned, non_blocking=True)
        out = self.step_device()
        self.host_logits.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.host_logits

    # ---- pipelined end-to-end call ------------------------------------------------------------------------------------
    def _make_slots(self):
        """Two input slots, each with its own captured graph, logits and pinned result buffer, plus a copy-in and a
        copy-out stream: batch i+1 crosses PCIe while batch i computes and batch i-1's logits go back."""
        dev = self.net.device
        self.h2d_stream, self.d2h_stream = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.slots = []
        for k in range(2):
            x = self.x_dev if k == 0 else torch.empty_like(self.x_dev)
            if k == 0:
                graph, logits = self.graph, self.logits
            else:
                x.copy_(self.x_dev)
                graph, logits = self.net.capture(x, fold=self.fold)
            n, c = logits.shape
            self.slots.append({
                "x": x, "graph": graph, "logits": logits,
                "all": self.all_logits if k == 0 else torch.empty_like(self.all_logits),
                "host": self.host_logits if k == 0 else torch.empty((n * self.world, c), dtype=torch.float32).pin_memory(),
                "in_ready": torch.cuda.Event(), "in_free": torch.cuda.Event(), "out_ready": torch.cuda.Event(), "host_ready": torch.cuda.Event(),
                "busy": False})

    def run_stream(self, batches):
        """Public streaming call: an iterable of pinned host fp32 NCHW batches in, one host logits array (all ranks' rows)
        out per batch, in order.  The returned array of batch i is valid until batch i+2 is submitted."""
        if self.slots is None:
            self._make_slots()
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
            out = s["logits"]
            if self.world > 1:
                gather_logits(s["logits"], self.world, s["all"])
                out = s["all"]
            s["out_ready"].record(compute)
            with torch.cuda.stream(self.d2h_stream):
                self.d2h_stream.wait_event(s["out_ready"])
                s["host"].copy_(out, non_blocking=True)
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
