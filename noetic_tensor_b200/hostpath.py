"""The fused forward for callers whose logits live in HOST memory.

Rows are independent, so host batches are streamed through the GPU in row chunks: while chunk i
is reduced on the compute stream, chunk i+1 crosses PCIe on a copy stream into the other of two
device slots, and the per-row results of chunk i−1 go back to pinned host memory. The device
never holds more than two chunks. All arithmetic is libnrl.so's; this file only moves bytes.

With a byte mask the link carries only what the forward reads (`packed=True`, the default): host
threads keep one liveness bit per 8-element vector and the logits, reference logits and mask
bytes of the live vectors (nrl_host_pack), and a kernel puts them back in place on the device
(nrl_unpack_rows). A chunk whose live vectors outgrow the staging buffers is uploaded whole.

`run_mapped` needs no staging at all: pinned host memory is mapped into the device's address
space, so the masked forward streams the mask from it in place and fetches only the vectors the
mask allows, each once, over the host link; no host thread touches the rows.

`run_hybrid` does both at once on two shares of the rows: the mapped path is bound by the number
of small reads the link keeps in flight, the packed path by the host's cores and memory, so the
two add up to more than either.
"""
import ctypes as C
import os
import threading

import torch

from . import capi, ops


def bind_host_thread_near(device):
    """Restricts the calling process to the CPUs next to `device` on the PCIe tree (the
    `local_cpulist` the kernel publishes for the GPU's PCI function), so that host buffers it then
    allocates and first touches land in the memory of that NUMA node: a kernel or a copy that reads
    them does not cross the socket interconnect. Returns the CPU set, or None when the topology is
    not visible (a container without /sys, a single-node host): nothing is changed then.
    The narrowing lasts until the caller undoes it: `os.sched_setaffinity(0, previous)` with the
    set `os.sched_getaffinity(0)` gave before the call, or use `host_threads_near` below."""
    try:
        p = torch.cuda.get_device_properties(torch.device(device))
        addr = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{addr}/local_cpulist") as fh:
            text = fh.read().strip()
        cpus = set()
        for part in text.split(","):
            if part:
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed or allowed == os.sched_getaffinity(0):
            return None
        os.sched_setaffinity(0, allowed)
        return allowed
    except Exception:
        return None


class host_threads_near:
    """`with host_threads_near(device):` — `bind_host_thread_near` for the block, the process's
    previous CPU affinity restored on leaving it."""

    def __init__(self, device):
        self.device = device

    def __enter__(self):
        self.previous = os.sched_getaffinity(0)
        self.cpus = bind_host_thread_near(self.device)
        return self.cpus

    def __exit__(self, *exc):
        if self.cpus is not None:
            os.sched_setaffinity(0, self.previous)
        return False


def default_host_threads():
    """Host threads one rank may use for packing: the CPUs this process may run on, shared evenly
    among the ranks of this host (LOCAL_WORLD_SIZE, as torchrun sets it), at most 32."""
    try:
        cpus = len(os.sched_getaffinity(0))
    except AttributeError:
        cpus = os.cpu_count() or 1
    local_world = max(1, int(os.environ.get("LOCAL_WORLD_SIZE", "1") or 1))
    return max(1, min(cpus // local_world, 32))


class HostForward:
    def __init__(self, V, dtype, *, chunk_rows=512, ref=True, mask=True, device="cuda:0", packed=True, live_fraction=0.25, threads=None):
        self.dev = torch.device(device)
        self.V, self.dtype, self.chunk = V, dtype, chunk_rows
        self.has_ref, self.has_mask = ref, mask
        self.packed = bool(packed and mask and V % 8 == 0 and V <= 262144)
        self.threads = int(threads or default_host_threads())
        self.words = (V // 8 + 63) // 64
        self.capacity = max(1, int(chunk_rows * (V // 8) * live_fraction))  # live vectors a chunk's staging buffers hold
        mk = lambda dt, *shape: torch.empty(*shape, dtype=dt, device=self.dev)
        pin = lambda dt, *shape: torch.empty(*shape, dtype=dt).pin_memory()
        self.slots = []
        for _ in range(2):
            s = dict(x=mk(dtype, chunk_rows, V), u=mk(torch.float32, chunk_rows))
            if ref:
                s["r"] = mk(dtype, chunk_rows, V)
            if mask:
                s["m"] = mk(torch.uint8, chunk_rows, V)
            if self.packed:
                for where, make in (("h", pin), ("d", mk)):
                    s[where + "_words"] = make(torch.int64, chunk_rows, self.words)
                    s[where + "_off"] = make(torch.int32, chunk_rows + 1)
                    s[where + "_px"] = make(dtype, self.capacity, 8)
                    if ref:
                        s[where + "_pr"] = make(dtype, self.capacity, 8)
                    s[where + "_pm"] = make(torch.int64, self.capacity)
                s["staged"] = torch.cuda.Event()  # the copies out of this slot's pinned staging buffers have finished
            s["ready"] = torch.cuda.Event()
            s["free"] = torch.cuda.Event()
            self.slots.append(s)
        self.packed_chunks = self.whole_chunks = 0
        self.copy_stream = torch.cuda.Stream(self.dev)
        self.back_stream = torch.cuda.Stream(self.dev)

    def bytes_per_row(self):
        """(host→device bytes of a row uploaded whole, device→host bytes of its results); what a
        call actually sent is in `h2d_bytes` after it."""
        e = torch.empty(0, dtype=self.dtype).element_size()
        return self.V * (e * (2 if self.has_ref else 1) + (1 if self.has_mask else 0)) + 4, 4 * 4 + 1

    def _pack(self, s, i, logits, ref, mask, r0, r1):
        """Host threads compact rows [r0, r1) into the slot's pinned staging buffers. Returns the
        number of live vectors, or None when they do not fit (the chunk is then uploaded whole)."""
        if i >= 2:
            s["staged"].synchronize()  # the previous copies out of these staging buffers are done
        a = capi.PackArgs()
        a.struct_size = C.sizeof(a)
        a.dtype, a.V, a.threads, a.rows, a.capacity = (capi.F32 if self.dtype == torch.float32 else capi.BF16), self.V, self.threads, r1 - r0, self.capacity
        esize = logits.element_size()
        a.logits = logits.data_ptr() + r0 * self.V * esize
        a.ref_logits = ref.data_ptr() + r0 * self.V * esize if self.has_ref else None
        a.allow_mask = mask.data_ptr() + r0 * self.V
        a.live_words, a.row_offset = s["h_words"].data_ptr(), s["h_off"].data_ptr()
        a.packed_logits, a.packed_mask = s["h_px"].data_ptr(), s["h_pm"].data_ptr()
        a.packed_ref = s["h_pr"].data_ptr() if self.has_ref else None
        rc = capi.lib().nrl_host_pack(C.byref(a))
        if rc == capi.E_WORKSPACE:
            return None
        capi.check(rc, "nrl_host_pack")
        return int(a.live_vectors)

    def _unpack(self, s, n):
        a = capi.UnpackArgs()
        a.struct_size = C.sizeof(a)
        a.dtype, a.V, a.rows = (capi.F32 if self.dtype == torch.float32 else capi.BF16), self.V, n
        a.live_words, a.row_offset = s["d_words"].data_ptr(), s["d_off"].data_ptr()
        a.packed_logits, a.packed_mask = s["d_px"].data_ptr(), s["d_pm"].data_ptr()
        a.packed_ref = s["d_pr"].data_ptr() if self.has_ref else 0
        a.logits, a.allow_mask = s["x"].data_ptr(), s["m"].data_ptr()
        a.ref_logits = s["r"].data_ptr() if self.has_ref else 0
        capi.check(capi.lib().nrl_unpack_rows(C.byref(a), C.c_void_p(self.copy_stream.cuda_stream)), "nrl_unpack_rows")

    def run_mapped(self, logits, uniforms, ref=None, mask=None, out=None, chunk_rows=2048, mask_by_copy=True, mask_bits=None, first_chunk_rows=None, pack_bits_on_host=False):
        """The same results as `run`, the kernel reading the pinned host logits (and reference) in
        place. With `mask_by_copy` the byte mask, which is read whole, goes up by copies in
        `chunk_rows`-row chunks one chunk ahead of the kernel (the copy engine moves it faster than
        loads over the link do); otherwise one launch reads everything in place. A caller that holds
        bit-packed masks passes `mask_bits` (pinned int32 [rows, ceil(V/32)], bit v of a row = bit
        v mod 32 of word v / 32) instead of `mask`: V/8 bytes per row go up and the kernels read
        the bits as they are (NRL_FWD_MASK_BITS). `first_chunk_rows` makes the first chunk smaller:
        its mask copy is the one nothing overlaps. With `pack_bits_on_host` a BYTE mask is turned
        into bits by host threads chunk by chunk (nrl_host_pack_bits, one chunk ahead of the kernel)
        so that only V/8 mask bytes per row cross the link; the results are the byte mask's."""
        if not self.has_mask:
            mask = mask_bits = None
        if mask is None and mask_bits is None:
            # every logit is read: copies move whole rows about twice as fast as loads over the link
            return self.run(logits, uniforms, ref=ref, mask=None, out=out)
        rows = logits.shape[0]
        pin = lambda dt: torch.empty(rows, dtype=dt).pin_memory()
        if out is None:
            out = dict(tokens=pin(torch.int32), logp=pin(torch.float32), kl=pin(torch.float32), entropy=pin(torch.float32), status=pin(torch.uint8))
        compute = torch.cuda.current_stream(self.dev)
        u = uniforms.to(self.dev, non_blocking=True)
        ref = ref if self.has_ref else None
        mask = mask if self.has_mask else None
        host_pack = bool(pack_bits_on_host and mask is not None and mask_bits is None)
        byte_mask = mask
        if host_pack:  # bits are made per chunk below; `mask_bits` stands for "the kernels get bits"
            words = (self.V + 31) // 32
            n_stage = min(chunk_rows, rows)
            if getattr(self, "_host_bits", None) is None or self._host_bits[0].shape[0] < n_stage or self._host_bits[0].shape[1] != words:
                self._host_bits = [torch.empty(n_stage, words, dtype=torch.int32).pin_memory() for _ in range(2)]
                self._host_bits_copied = [torch.cuda.Event() for _ in range(2)]
            mask_bits = self._host_bits[0]  # only its shape is used before the loop
        if mask_bits is not None:
            mask, mask_by_copy = mask_bits, True
            if getattr(self, "_mapped_bits", None) is None or self._mapped_bits[0].shape[0] < min(chunk_rows, rows) or self._mapped_bits[0].shape[1] != mask_bits.shape[1]:
                self._mapped_bits = [torch.empty(min(chunk_rows, rows), mask_bits.shape[1], dtype=torch.int32, device=self.dev) for _ in range(2)]
        by_copy = mask_by_copy and mask is not None
        if not by_copy:
            chunk_rows = rows
        else:
            if getattr(self, "_mapped_events", None) is None:
                self._mapped_events = [(torch.cuda.Event(), torch.cuda.Event()) for _ in range(2)]
            if mask_bits is None and (getattr(self, "_mapped_masks", None) is None or self._mapped_masks[0].shape[0] < min(chunk_rows, rows)):
                self._mapped_masks = [torch.empty(min(chunk_rows, rows), self.V, dtype=torch.uint8, device=self.dev) for _ in range(2)]
        results = []
        starts = list(range(0, rows, chunk_rows))
        if by_copy and first_chunk_rows and first_chunk_rows < min(chunk_rows, rows):
            starts = [0] + list(range(first_chunk_rows, rows, chunk_rows))
        for i, r0 in enumerate(starts):
            r1 = starts[i + 1] if i + 1 < len(starts) else rows
            m = mask[r0:r1] if mask is not None else None
            if by_copy:
                ready, free = self._mapped_events[i % 2]
                with torch.cuda.stream(self.copy_stream):
                    if i >= 2:
                        self.copy_stream.wait_event(free)  # the kernel that read this buffer has finished
                    if host_pack:
                        stage = self._host_bits[i % 2][: r1 - r0]
                        if i >= 2:
                            self._host_bits_copied[i % 2].synchronize()  # the copy out of this staging buffer is done
                        capi.check(capi.lib().nrl_host_pack_bits(r1 - r0, self.V, byte_mask.data_ptr() + r0 * self.V, stage.data_ptr(), self.threads), "nrl_host_pack_bits")
                        m, bits = None, self._mapped_bits[i % 2][: r1 - r0]
                        bits.copy_(stage, non_blocking=True)
                        self._host_bits_copied[i % 2].record(self.copy_stream)
                    elif mask_bits is not None:
                        m, bits = None, self._mapped_bits[i % 2][: r1 - r0]
                        bits.copy_(mask_bits[r0:r1], non_blocking=True)
                    else:
                        m, bits = self._mapped_masks[i % 2][: r1 - r0], None
                        m.copy_(mask[r0:r1], non_blocking=True)
                    ready.record(self.copy_stream)
                compute.wait_event(ready)
            else:
                bits = None
            f = ops.row_forward(logits[r0:r1], ref_logits=None if ref is None else ref[r0:r1], allow=m, allow_bits=bits, uniforms=u[r0:r1], device=self.dev)
            if by_copy:
                free.record(compute)
            for name in ("tokens", "logp", "kl", "entropy", "status"):
                t = getattr(f, name)
                if t is not None:
                    out[name][r0:r1].copy_(t, non_blocking=True)
            results.append(f)
        compute.synchronize()
        self.copy_stream.synchronize()
        return out

    def run(self, logits, uniforms, ref=None, mask=None, out=None):
        """logits/ref [rows, V], mask [rows, V] u8, uniforms [rows]: pinned host tensors. Returns
        pinned host tensors tokens (i32), logp, kl, entropy (f32) and status (u8), complete on return."""
        if (self.has_mask and mask is None) or (self.has_ref and ref is None):
            raise ValueError("HostForward was built for rows with a mask / a reference stream: pass them")
        rows = logits.shape[0]
        if out is None:
            pin = lambda dt: torch.empty(rows, dtype=dt).pin_memory()
            out = dict(tokens=pin(torch.int32), logp=pin(torch.float32), kl=pin(torch.float32), entropy=pin(torch.float32), status=pin(torch.uint8))
        compute = torch.cuda.current_stream(self.dev)
        done = []
        self.h2d_bytes = 0  # bytes this call sends to the device
        self.live_vectors = 0  # 8-element vectors the mask allows, over the packed chunks of this call
        esize = logits.element_size()
        for i, r0 in enumerate(range(0, rows, self.chunk)):
            r1 = min(rows, r0 + self.chunk)
            n = r1 - r0
            s = self.slots[i % 2]
            live = self._pack(s, i, logits, ref, mask, r0, r1) if self.packed else None
            with torch.cuda.stream(self.copy_stream):
                if i >= 2:
                    self.copy_stream.wait_event(s["free"])  # the kernel that read this slot has finished
                s["u"][:n].copy_(uniforms[r0:r1], non_blocking=True)
                if live is not None:
                    s["d_words"][:n].copy_(s["h_words"][:n], non_blocking=True)
                    s["d_off"][: n + 1].copy_(s["h_off"][: n + 1], non_blocking=True)
                    s["d_px"][:live].copy_(s["h_px"][:live], non_blocking=True)
                    if self.has_ref:
                        s["d_pr"][:live].copy_(s["h_pr"][:live], non_blocking=True)
                    s["d_pm"][:live].copy_(s["h_pm"][:live], non_blocking=True)
                    s["staged"].record(self.copy_stream)
                    self._unpack(s, n)
                    self.packed_chunks += 1
                    self.live_vectors += live
                    self.h2d_bytes += n * 4 + n * self.words * 8 + (n + 1) * 4 + live * (8 * esize * (2 if self.has_ref else 1) + 8)
                else:
                    s["x"][:n].copy_(logits[r0:r1], non_blocking=True)
                    if self.has_ref:
                        s["r"][:n].copy_(ref[r0:r1], non_blocking=True)
                    if self.has_mask:
                        s["m"][:n].copy_(mask[r0:r1], non_blocking=True)
                    self.whole_chunks += 1
                    self.h2d_bytes += n * self.bytes_per_row()[0]
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

    def run_hybrid(self, logits, uniforms, ref=None, mask=None, out=None, packed_share=0.375, mapped_chunk_rows=1184, packed_threads=None):
        """The rows split in two: the first share through `run_mapped` (the kernel fetches the live
        vectors over the link; host threads turn the byte mask into bits), the last `packed_share`
        through `run` (host threads pack the live vectors, copies move them) on a second Python
        thread and a second CUDA stream, at the same time. Same results as either (every row is
        computed by the same kernels on the same values). `packed_threads` of this object's host
        threads (half of them by default) go to the packing, the rest to the bit masks. Measured on
        a B200 host with 16 cores: 3/8 of the rows packed by 8 threads gave the most."""
        if not (self.has_mask and self.packed) or mask is None:
            return self.run_mapped(logits, uniforms, ref=ref, mask=mask, out=out)
        rows = logits.shape[0]
        n_packed = int(rows * packed_share) // self.chunk * self.chunk
        n_mapped = rows - n_packed
        if n_packed == 0 or n_mapped == 0:
            return self.run_mapped(logits, uniforms, ref=ref, mask=mask, out=out, chunk_rows=mapped_chunk_rows, first_chunk_rows=min(512, mapped_chunk_rows), pack_bits_on_host=True)
        if out is None:
            pin = lambda dt: torch.empty(rows, dtype=dt).pin_memory()
            out = dict(tokens=pin(torch.int32), logp=pin(torch.float32), kl=pin(torch.float32), entropy=pin(torch.float32), status=pin(torch.uint8))
        pt = int(packed_threads or max(1, self.threads // 2))
        twin = getattr(self, "_twin", None)
        if twin is None or twin.threads != pt:
            twin = self._twin = HostForward(self.V, self.dtype, chunk_rows=self.chunk, ref=self.has_ref, mask=True, device=self.dev, packed=True, threads=pt)
            self._twin_stream = torch.cuda.Stream(self.dev)
        a, b = slice(0, n_mapped), slice(n_mapped, rows)
        part = lambda t, s: None if t is None else t[s]
        failure = []

        def packed_side():
            try:
                torch.cuda.set_device(self.dev)
                with torch.cuda.stream(self._twin_stream):
                    twin.run(logits[b], uniforms[b], ref=part(ref, b), mask=mask[b], out={k: v[b] for k, v in out.items()})
            except BaseException as e:  # handed to the caller below
                failure.append(e)

        worker = threading.Thread(target=packed_side)
        worker.start()
        keep = self.threads
        self.threads = max(1, keep - pt)
        try:
            self.run_mapped(logits[a], uniforms[a], ref=part(ref, a), mask=mask[a], out={k: v[a] for k, v in out.items()}, chunk_rows=mapped_chunk_rows,
                            first_chunk_rows=min(512, mapped_chunk_rows), pack_bits_on_host=True)
        finally:
            self.threads = keep
            worker.join()
        if failure:
            raise failure[0]
        self.h2d_bytes, self.live_vectors = twin.h2d_bytes, twin.live_vectors
        return out
