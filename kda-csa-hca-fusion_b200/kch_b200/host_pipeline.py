"""Host-resident batches through the stack with the PCIe copies hidden behind the kernels.

The reference keeps its tensors wherever the caller put them and has no notion of streams.  A caller whose
hidden states live in host memory pays one host->device copy before and one device->host copy after every
forward pass; at the benchmark size those copies (2 x 537 MB) cost about a third of the pass itself.
``HostPipeline`` runs a sequence of passes with three CUDA streams: while pass ``i`` computes, the input of
pass ``i+1`` is uploaded into the other of two device buffers and the output of pass ``i-1`` is downloaded.
Every copy still happens, once per pass; only the first upload and the last download are exposed.

Under tensor parallelism (``tp=`` a ``TPContext`` of more than one rank) every rank needs the whole batch on its GPU, but
it does not have to come over every rank's PCIe link: each rank uploads its 1/N run of the flattened ``[B*T]`` rows, the
runs are all-gathered over NVLink (one collective per pass, on the compute stream), and each rank downloads its run of
the output only -- the host moves one copy of the batch per pass instead of N.
"""
from __future__ import annotations

import torch


class HostPipeline:
    def __init__(self, model, device=None, tp=None):
        self.model = model
        self.tp = tp if (tp is not None and tp.world > 1) else None
        self._xfull = None
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("HostPipeline requires a CUDA device; there is no CPU path")
        self._up = torch.cuda.Stream(self.device)
        self._down = torch.cuda.Stream(self.device)
        self._xd = [None, None]

    @torch.no_grad()
    def run(self, inputs, outputs, *, reset_state=True):
        """``inputs[i]`` (pinned host ``[B,T,d]``) -> ``outputs[i]`` (pinned host, same shape).  Passes are
        independent prefill passes when ``reset_state`` (the KDA state is cleared before each).  With ``tp`` every rank
        passes the same ``inputs`` and finds ITS run of rows filled in ``outputs[i]`` (the runs of all ranks make up
        the whole output)."""
        if len(inputs) != len(outputs):
            raise ValueError(f"HostPipeline.run: {len(inputs)} inputs but {len(outputs)} outputs")
        dev = self.device
        compute = torch.cuda.current_stream(dev)
        n = len(inputs)
        uploaded = [torch.cuda.Event() for _ in range(n)]
        computed = [torch.cuda.Event() for _ in range(n)]
        self._up.wait_stream(compute)
        self._down.wait_stream(compute)

        tp = self.tp

        def my_rows(t):                          # this rank's run of the flattened rows of a host tensor
            flat = t.reshape(-1, t.shape[-1])
            if flat.shape[0] % tp.world != 0:
                raise ValueError(f"HostPipeline.run: {flat.shape[0]} rows do not divide over {tp.world} ranks")
            per = flat.shape[0] // tp.world
            return flat[tp.rank * per:(tp.rank + 1) * per]

        def upload(i):
            x = inputs[i] if tp is None else my_rows(inputs[i])
            slot = i % 2
            if self._xd[slot] is None or self._xd[slot].shape != x.shape or self._xd[slot].dtype != x.dtype:
                self._xd[slot] = torch.empty(x.shape, dtype=x.dtype, device=dev)
                # allocated from the compute stream's pool but written on the upload stream: tell the allocator,
                # so that a replaced buffer is not handed out again while an upload into it is still in flight
                self._xd[slot].record_stream(self._up)
            with torch.cuda.stream(self._up):
                if i >= 2:
                    self._up.wait_event(computed[i - 2])        # the pass that read this buffer has finished
                self._xd[slot].copy_(x, non_blocking=True)
                uploaded[i].record(self._up)

        if n:
            upload(0)
        for i in range(n):
            if i + 1 < n:
                upload(i + 1)
            compute.wait_event(uploaded[i])
            if reset_state:
                self.model.reset_state()
            if tp is None:
                xin = self._xd[i % 2]
            else:
                import torch.distributed as dist
                full_shape = inputs[i].shape
                if self._xfull is None or self._xfull.shape != full_shape or self._xfull.dtype != inputs[i].dtype:
                    self._xfull = torch.empty(full_shape, dtype=inputs[i].dtype, device=dev)
                dist.all_gather_into_tensor(self._xfull.view(-1, full_shape[-1]), self._xd[i % 2], group=tp.group)
                xin = self._xfull
            y = self.model(xin)
            computed[i].record(compute)
            with torch.cuda.stream(self._down):
                self._down.wait_event(computed[i])
                if tp is None:
                    outputs[i].copy_(y, non_blocking=True)
                else:
                    my_rows(outputs[i]).copy_(my_rows(y), non_blocking=True)
            y.record_stream(self._down)
        compute.wait_stream(self._down)
        self._raise_on_device_status()
        return outputs

    def _raise_on_device_status(self):
        """The kernels' bounded waits report through a sticky status word; once it is set, later kernels return
        without writing their outputs.  Read it where the host waits anyway (the downloads have to complete
        before the caller may use `outputs`), and turn it into an exception instead of silent garbage."""
        from . import _lib
        with torch.cuda.device(self.device):
            _lib.raise_on_device_status("HostPipeline.run")
