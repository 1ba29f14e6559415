"""The fused forward for callers whose logits live in HOST memory.

Rows are independent, so host batches are streamed through the GPU in row chunks: while chunk i
is reduced on the compute stream, chunk i+1 crosses PCIe on a copy stream into the other of two
device slots, and the per-row results of chunk i−1 go back to pinned host memory. The device
never holds more than two chunks. All arithmetic is libnrl.so's; this file only moves bytes.
"""
import torch

from . import ops


class HostForward:
    def __init__(self, V, dtype, *, chunk_rows=512, ref=True, mask=True, device="cuda:0"):
        self.dev = torch.device(device)
        self.V, self.dtype, self.chunk = V, dtype, chunk_rows
        self.has_ref, self.has_mask = ref, mask
        mk = lambda dt, *shape: torch.empty(*shape, dtype=dt, device=self.dev)
        self.slots = []
        for _ in range(2):
            s = dict(x=mk(dtype, chunk_rows, V), u=mk(torch.float32, chunk_rows))
            if ref:
                s["r"] = mk(dtype, chunk_rows, V)
            if mask:
                s["m"] = mk(torch.uint8, chunk_rows, V)
            s["ready"] = torch.cuda.Event()
            s["free"] = torch.cuda.Event()
            self.slots.append(s)
        self.copy_stream = torch.cuda.Stream(self.dev)
        self.back_stream = torch.cuda.Stream(self.dev)

    def bytes_per_row(self):
        e = torch.empty(0, dtype=self.dtype).element_size()
        return self.V * (e * (2 if self.has_ref else 1) + (1 if self.has_mask else 0)) + 4, 4 * 4 + 1

    def run(self, logits, uniforms, ref=None, mask=None, out=None):
        """logits/ref [rows, V], mask [rows, V] u8, uniforms [rows]: pinned host tensors. Returns
        pinned host tensors tokens (i32), logp, kl, entropy (f32) and status (u8), complete on return."""
        rows = logits.shape[0]
        if out is None:
            pin = lambda dt: torch.empty(rows, dtype=dt).pin_memory()
            out = dict(tokens=pin(torch.int32), logp=pin(torch.float32), kl=pin(torch.float32), entropy=pin(torch.float32), status=pin(torch.uint8))
        compute = torch.cuda.current_stream(self.dev)
        done = []
        for i, r0 in enumerate(range(0, rows, self.chunk)):
            r1 = min(rows, r0 + self.chunk)
            n = r1 - r0
            s = self.slots[i % 2]
            with torch.cuda.stream(self.copy_stream):
                if i >= 2:
                    self.copy_stream.wait_event(s["free"])  # the kernel that read this slot has finished
                s["x"][:n].copy_(logits[r0:r1], non_blocking=True)
                s["u"][:n].copy_(uniforms[r0:r1], non_blocking=True)
                if self.has_ref:
                    s["r"][:n].copy_(ref[r0:r1], non_blocking=True)
                if self.has_mask:
                    s["m"][:n].copy_(mask[r0:r1], non_blocking=True)
                s["ready"].record(self.copy_stream)
            compute.wait_event(s["ready"])
            f = ops.row_forward(s["x"][:n], ref_logits=s["r"][:n] if self.has_ref else None, allow=s["m"][:n] if self.has_mask else None, uniforms=s["u"][:n])
            s["free"].record(compute)
            ev = torch.cuda.Event()
            ev.record(compute)
            with torch.cuda.stream(self.back_stream):
                self.back_stream.wait_event(ev)
                out["tokens"][r0:r1].copy_(f.tokens, non_blocking=True)
                out["logp"][r0:r1].copy_(f.logp, non_blocking=True)
                if f.kl is not None:
                    out["kl"][r0:r1].copy_(f.kl, non_blocking=True)
                out["entropy"][r0:r1].copy_(f.entropy, non_blocking=True)
                out["status"][r0:r1].copy_(f.status, non_blocking=True)
                for t in (f.tokens, f.logp, f.kl, f.entropy, f.status):
                    if t is not None:
                        t.record_stream(self.back_stream)
            done.append(f)
        self.back_stream.synchronize()
        compute.synchronize()
        return out
