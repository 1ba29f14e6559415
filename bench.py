#!/usr/bin/env python
"""Benchmark of the fused sample + log-prob + KL + entropy forward at the Llama-3 vocabulary.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("headline"): config 3 of the baseline — logits [S=8, B=32, T=1024, V=128256] bf16
~N(0,3) plus a log-Zipf(1.1) token prior, a U8 grammar mask per row (1–4 bands of width 64–4096
plus 1 % random tokens) — with a bf16 frozen-reference stream (policy + N(0, 0.05)), one uniform
per row. A step is one pass of the fused forward over the resident batch: every element of the
logits, the reference and the mask is read from HBM once (5 bytes per element). Inputs are
seeded synthetic data; the batch (tens of GB) is far larger than L2, so nothing is flushed
between steps. One rank per GPU, rows partitioned across ranks, no collective on the data path.

Prints one JSON line on stdout: the metric (rows/s over all ranks, device-timed, inputs resident),
`roofline` of the one kernel a step launches, `cpu_baseline` (the CPU oracle on a sample of the
rows), `e2e` (the same metric from pinned host memory through the host path, copies included),
`clocks` sampled while the timed region ran, and `extras` (backward, other configurations).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

V = 128256
S_FULL, B, T = 8, 32, 1024
ROWS_PER_SEED = B * T
BYTES_PER_ELEM = 2 + 2 + 1  # bf16 logits + bf16 reference + u8 mask: the algorithmic bytes per element
METRIC = "rows/s fused sample+logprob+KL+entropy, V=128256 bf16"
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per launch ÷ algorithmic bytes per launch, from the ncu capture summarised in
# profiles/ (None until a capture exists for the current kernel).
NCU_TRAFFIC_RATIO = 0.626  # profiles/row_fwd_grouped_bf16_ref_allow_4096rows.md: 1.6437 GB of DRAM traffic per 2.6267 GB algorithmic

def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.t0 = self.t1 = None

    def wait_first(self, limit=8.0):
        """nvidia-smi needs a second or two to come up on a box with many GPUs: wait for its first line."""
        t = time.perf_counter()
        while self.proc and not self.rows and time.perf_counter() - t < limit:
            time.sleep(0.02)

    def begin(self):
        self.t0 = time.perf_counter()

    def end(self):
        self.t1 = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([time.perf_counter()] + [c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        rows = self.rows
        if self.t0 is not None and self.t1 is not None:  # the samples that arrived while the region of interest ran
            rows = [r for r in rows if self.t0 <= r[0] <= self.t1 + 0.12]
        for r in (r[1:] for r in rows):
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def make_inputs(rows, seed, device):
    import torch

    from noetic_tensor_b200 import synth

    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    bias = synth.zipf_bias(V, 1.1, gen, device)
    logits = synth.normal_logits(rows, V, 3.0, torch.bfloat16, gen, device, bias=bias)
    ref = synth.perturbed(logits, 0.05, gen)
    mask = synth.grammar_masks(rows, V, gen, device)
    u = synth.uniforms(rows, gen, device)
    return logits, ref, mask, u


def necessary_bytes(mask, granule):
    """Bytes a launch over these rows cannot avoid moving when memory is fetched in aligned granules
    of `granule` bytes: the byte mask whole, plus every granule of the bf16 logits and of the bf16
    reference that holds at least one allowed token. Counted on the device, outside the timing."""
    rows, v = mask.shape
    elems = granule // 2
    live = 0
    for r0 in range(0, rows, 4096):
        m = mask[r0:r0 + 4096]
        live += int(m.view(m.shape[0], v // elems, elems).ne(0).any(dim=2).sum().item())
    return rows * v + 2 * live * granule


def close(a, b):
    """1e-5 relative or 1e-6 absolute, the path's tolerance; NaN equals NaN."""
    import torch

    a, b = a.double().cpu(), b.double().cpu()
    d = (a - b).abs()
    ok = (d <= 1e-6) | (d <= 1e-5 * b.abs()) | (a == b) | (torch.isnan(a) & torch.isnan(b))
    return int((~ok).sum().item())


def compare_with_resident(host_out, res, n):
    """Every row of a host path's results against the resident launch's: tokens that differ (the two
    run different decompositions of a row when the chunk sizes differ, so a uniform on a CDF step
    may fall either way), and log-prob / KL / entropy outside the tolerance on rows with the same token."""
    import torch

    tok_h, tok_r = host_out["tokens"][:n], res.tokens[:n].cpu()
    same = tok_h == tok_r
    bad = close(host_out["logp"][:n][same], res.logp[:n].cpu()[same]) + close(host_out["kl"][:n], res.kl[:n]) + close(host_out["entropy"][:n], res.entropy[:n])
    return {"rows": n, "tokens_differing": int((~same).sum().item()), "values_outside_tolerance": bad}


def cpu_reference_rows(logits_bits, ref_bits, allow, root, fast, threads):
    """The reference's own path for the same quantities on a row sample: sample_categorical
    (Gumbel-max, one ChaCha20 u64 per logit) + token_log_probs + reference_kl + categorical_entropy,
    each under the same additive −inf vocabulary mask. Returns seconds."""
    import numpy as np

    import oracle

    oracle.set_backend(fast, threads)
    rows = logits_bits.shape[0]
    shape = (1, 1, rows, V)
    add = np.where(allow != 0, 0.0, -np.inf).astype(np.float32)
    t0 = time.perf_counter()
    tok = oracle.sample_gumbel(logits_bits, 1.0, root, "bench", add_mask=add)
    vm = add.astype(np.float64)
    oracle.rl_eval(oracle.OP_TOKEN_LOG_PROBS, shape, logits=logits_bits, tokens=tok, vocab_mask=vm)
    oracle.rl_eval(oracle.OP_REFERENCE_KL, shape, logits=logits_bits, ref_logits=ref_bits, vocab_mask=vm)
    oracle.rl_eval(oracle.OP_ENTROPY, shape, logits=logits_bits, vocab_mask=vm)
    dt = time.perf_counter() - t0
    oracle.set_backend(False, 1)
    return dt


def host_sample(rows, seed):
    """A row sample of the workload on the host (bf16 bit patterns), for the CPU arms."""
    import numpy as np
    import torch

    g = torch.Generator()
    g.manual_seed(seed)
    perm = torch.randperm(V, generator=g)
    rank = torch.empty(V)
    rank[perm] = torch.arange(1, V + 1, dtype=torch.float32)
    bias = -1.1 * torch.log(rank)
    x = (torch.randn(rows, V, generator=g) * 3.0 + bias).to(torch.bfloat16)
    r = (x.float() + torch.randn(rows, V, generator=g) * 0.05).to(torch.bfloat16)
    m = torch.rand(rows, V, generator=g) < 0.01
    col = torch.arange(V)[None, :]
    nb = torch.randint(1, 5, (rows,), generator=g)
    for k in range(4):
        w = torch.randint(64, 4097, (rows, 1), generator=g)
        s0 = (torch.rand(rows, 1, generator=g) * (V - 4096)).long()
        m |= (nb > k)[:, None] & (col >= s0) & (col < s0 + w)
    bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)
    return bits(x), bits(r), m.to(torch.uint8).numpy()


_REF_ROWS = None


def _reference_init(rows, seed0):
    """A reference-arm process: its own rows of the workload, generated once, outside the timing."""
    global _REF_ROWS
    import multiprocessing as mp

    import torch

    torch.set_num_threads(1)
    ident = mp.current_process()._identity
    _REF_ROWS = host_sample(rows, seed0 + (ident[0] if ident else 0))


def _reference_worker(root):
    """Cpu(Reference), single thread, on this process's rows; returns its seconds."""
    xb, rb, al = _REF_ROWS
    return cpu_reference_rows(xb, rb, al, root, False, 1)


def run_reference(args):
    """The reference's own CPU path on the host cores. Rows are independent (the reference's seed
    axis never mixes), so the arm runs one Cpu(Reference) process per core, each on its own rows:
    that is every host thread the path can use. Cpu(Fast), the reference's threaded backend (all
    threads inside each op), is timed once beside it and noted."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import concurrent.futures as cf

    cores = os.cpu_count() or 1
    workers = max(1, min(cores, 64))
    rows_each = 8
    sample_rows = workers * rows_each
    with cf.ProcessPoolExecutor(max_workers=workers, initializer=_reference_init, initargs=(rows_each, 5000)) as pool:
        for _ in range(max(1, min(args.warmup, 1))):
            list(pool.map(_reference_worker, [1] * workers))
        times = []
        for i in range(args.steps):
            t0 = time.perf_counter()
            list(pool.map(_reference_worker, [2 + i] * workers))  # one job per process: each runs its own rows
            times.append(time.perf_counter() - t0)
    dt = sum(times) / len(times)
    value = sample_rows / dt
    xb, rb, al = host_sample(16, 1234)
    fast = 16 / cpu_reference_rows(xb, rb, al, 2, True, cores)
    line = {
        "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
        "config": {"workload": "config 3 [8,32,1024,128256] bf16 + U8 grammar mask + bf16 reference stream (headline)", "rows_per_step": sample_rows, "V": V},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": workers, "kind": "port",
                         "sample": f"{sample_rows} rows of the workload per step ({rows_each} per process, {workers} processes); C++ restatement of the "
                                   "reference's Cpu(Reference) op sequence (sample_categorical Gumbel-max + token_log_probs + reference_kl + categorical_entropy); "
                                   f"its threaded Cpu(Fast) backend on {cores} threads does {fast:.1f} rows/s on 16 rows; the Rust reference cannot be built here"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def _time(fn, iters=5, warm=3):
    import torch

    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def run_extras(dev, peak):
    """Secondary measurements on row slices of the other configurations (device-timed, inputs
    resident, each slice several GB so L2 holds none of it): not the headline, reported so that
    every kernel on the path has a number. bytes = algorithmic bytes of forward + backward."""
    import torch

    from noetic_tensor_b200 import capi, ops, synth

    gen = torch.Generator(device=dev)
    gen.manual_seed(77)
    res = {}

    def entry(rows, ms, nbytes, what):
        return {"what": what, "rows": rows, "ms": ms, "rows_per_s": rows / (ms * 1e-3), "GBps": nbytes / (ms * 1e-3) / 1e9, "frac_of_measured_peak": nbytes / (ms * 1e-3) / 1e9 / peak}

    # headline shape, forward + backward to d(logits)
    rows = 8192
    bias = synth.zipf_bias(V, 1.1, gen, dev)
    x = synth.normal_logits(rows, V, 3.0, torch.bfloat16, gen, dev, bias=bias)
    r = synth.perturbed(x, 0.05, gen)
    m = synth.grammar_masks(rows, V, gen, dev)
    u = synth.uniforms(rows, gen, dev)
    ones = torch.ones(rows, device=dev)
    d = torch.empty(rows, V, dtype=torch.float32, device=dev)

    def fwd_bwd():
        f = ops.row_forward(x, ref_logits=r, allow=m, uniforms=u)
        ops.row_backward(x, f, ref_logits=r, allow=m, g_logp=ones, g_kl=ones, g_ent=ones, out=d)

    res["headline_fwd_bwd"] = entry(rows, _time(fwd_bwd), rows * V * (5 + 5 + 4), "config 3 + reference: sample+logp+KL+entropy forward, then backward to f32 d(logits)")
    f = ops.row_forward(x, ref_logits=r, allow=m, uniforms=u)
    res["headline_bwd_only"] = entry(rows, _time(lambda: ops.row_backward(x, f, ref_logits=r, allow=m, g_logp=ones, g_kl=ones, g_ent=ones, out=d)), rows * V * (5 + 4),
                                     "row backward alone (reads logits, reference, mask; writes f32 gradients)")
    res["unmasked_fwd"] = entry(rows, _time(lambda: ops.row_forward(x, ref_logits=r, uniforms=u)), rows * V * 4, "same logits and reference without a mask: every byte is read")
    # the same rows with the mask bit-packed (one bit per token, read by the kernels as it is)
    import numpy as np
    bits = torch.from_numpy(np.packbits(m.cpu().numpy(), axis=1, bitorder="little").view(np.int32)).to(dev)
    fb = ops.row_forward(x, ref_logits=r, allow_bits=bits, uniforms=u)
    same = bool(torch.equal(fb.tokens, f.tokens) and torch.equal(fb.logp.view(torch.int32), f.logp.view(torch.int32)))
    res["headline_fwd_bit_masks"] = entry(rows, _time(lambda: ops.row_forward(x, ref_logits=r, allow_bits=bits, uniforms=u)), rows * V * 4 + rows * (V // 8),
                                          "headline forward with bit-packed masks (NRL_FWD_MASK_BITS): 4 B of logits + 1 bit of mask per token")
    res["headline_fwd_bit_masks"]["same_bits_as_byte_masks"] = same

    def fwd_bwd_bits():
        g = ops.row_forward(x, ref_logits=r, allow_bits=bits, uniforms=u)
        ops.row_backward(x, g, ref_logits=r, allow_bits=bits, g_logp=ones, g_kl=ones, g_ent=ones, out=d)

    res["headline_fwd_bwd_bit_masks"] = entry(rows, _time(fwd_bwd_bits), rows * V * (4 + 4 + 4) + 2 * rows * (V // 8), "forward + backward with bit-packed masks")
    del x, r, m, d, f, fb, bits

    # config 4: one PPO step, V = 151936, forward + token losses + backward
    V4, S4, B4, T4 = 151936, 1, 32, 256
    rows = S4 * B4 * T4
    x = synth.normal_logits(rows, V4, 2.5, torch.bfloat16, gen, dev)
    r = synth.perturbed(x, 0.05, gen)
    u = synth.uniforms(rows, gen, dev)
    tok = ops.row_forward(x, uniforms=u, want_entropy=False).tokens
    f0 = ops.row_forward(x, ref_logits=r, tokens=tok)
    old = (f0.logp + 0.02 * torch.randn(rows, generator=gen, device=dev)).reshape(S4, B4, T4).contiguous()
    adv = synth.group_relative_advantages(S4, B4, 8, 0.3, gen, dev)
    d = torch.empty(rows, V4, dtype=torch.float32, device=dev)
    up = torch.ones(S4, device=dev)
    launches0 = capi.lib().nrl_launch_count()

    coef = [torch.ones(S4, device=dev), torch.full((S4,), 0.04, device=dev), torch.full((S4,), -0.01, device=dev)]

    def ppo_step():
        f = ops.row_forward(x, ref_logits=r, tokens=tok)
        o = ops.token_objective(capi.LOSS_PPO, f.logp.reshape(S4, B4, T4), capi.REDUCE_TOKEN_MEAN, other=old, weights=adv, clip_low=0.2, clip_high=0.2, clamp=20.0,
                                kl=f.kl.reshape(S4, B4, T4), entropy=f.entropy.reshape(S4, B4, T4), up_policy=coef[0], up_kl=coef[1], up_entropy=coef[2])
        ops.row_backward(x, f, ref_logits=r, g_logp=o.g_logp.reshape(-1), g_kl=o.g_kl.reshape(-1), g_ent=o.g_ent.reshape(-1), out=d)
        return o.policy, o.kl, o.entropy

    ms = _time(ppo_step)
    res["ppo_step_config4"] = entry(rows, ms, rows * V4 * (4 + 4 + 4), "config 4 slice [1,32,256,151936] bf16 + reference: PPO-clip 0.2 + 0.04 KL − 0.01 entropy, forward + backward to f32 d(logits)")
    res["ppo_step_config4"]["launches_per_step"] = (capi.lib().nrl_launch_count() - launches0) // 8
    del x, r, d, f0

    # config 2: dense f32 sampling + backward of the sampled tokens' log-probs
    V2, rows = 32000, 32768
    x = synth.normal_logits(rows, V2, 2.0, torch.float32, gen, dev)
    u = synth.uniforms(rows, gen, dev)
    ones = torch.ones(rows, device=dev)
    d = torch.empty(rows, V2, dtype=torch.float32, device=dev)

    def cfg2():
        f = ops.row_forward(x, uniforms=u)
        ops.row_backward(x, f, g_logp=ones, out=d)

    res["dense_f32_config2"] = entry(rows, _time(cfg2), rows * V2 * (4 + 4 + 4), "config 2 slice [rows,32000] f32, no mask: sample+logp+entropy forward, backward of the sum of sampled log-probs")
    del x, d

    # config 5: extreme sparse masks at V = 262144
    V5, rows = 262144, 4096
    x = synth.normal_logits(rows, V5, 4.0, torch.bfloat16, gen, dev)
    m, idx = synth.sparse_masks(rows, V5, gen, dev)
    shift = torch.zeros(rows, V5, dtype=torch.bfloat16, device=dev)
    live = idx >= 0
    rr = torch.arange(rows, device=dev)[:, None].expand(rows, 8)
    x[rr[live], idx[live]] -= 30.0
    r = synth.perturbed(x, 0.1, gen)
    del shift
    u = synth.uniforms(rows, gen, dev)
    ones = torch.ones(rows, device=dev)
    d = torch.empty(rows, V5, dtype=torch.float32, device=dev)

    def cfg5():
        f = ops.row_forward(x, ref_logits=r, allow=m, uniforms=u)
        ops.row_backward(x, f, ref_logits=r, allow=m, g_logp=ones, g_kl=ones, out=d)

    res["sparse_config5"] = entry(rows, _time(cfg5), rows * V5 * (5 + 5 + 4), "config 5 slice [rows,262144] bf16 + reference + masks allowing 1-8 tokens: masked sample+logp+KL forward + backward")
    del x, r, m, d

    # the pre-training loss on the same kernels: masked cross-entropy at V = 128256, forward + backward
    from noetic_tensor_b200 import loss as nloss

    S6, B6, T6 = 2, 4, 1024
    rows = S6 * B6 * T6
    x = synth.normal_logits(rows, V, 3.0, torch.bfloat16, gen, dev).reshape(S6, B6, T6, V)
    tg = torch.randint(0, V, (S6, B6, T6), generator=gen, device=dev)
    mk = (torch.rand(S6, B6, T6, generator=gen, device=dev) < 0.9).float()

    def ce_step():
        l = nloss.masked_cross_entropy(x, tg, mk)
        return l.backward()

    # the reference's own sampler on the device (Gumbel-max, one ChaCha20 u64 per logit): arithmetic-bound
    xs, ms_ = x.reshape(rows, V)[:4096], synth.grammar_masks(4096, V, gen, dev)
    seed = bytes(range(32))
    t_g = _time(lambda: ops.sample_gumbel(xs, seed, allow=ms_))
    res["reference_gumbel_sampler"] = entry(4096, t_g, 4096 * V * 3, "nrl_sample_gumbel on 4096 headline-shaped rows: tokens identical to the reference's sample_categorical for the same ChaCha20 seed (bytes = logits + mask; the kernel is bound by ChaCha20 and f64 logarithms, not by HBM)")
    del xs, ms_
    res["masked_cross_entropy_fwd_bwd"] = entry(rows, _time(ce_step), rows * V * (2 + 2 + 4), "nn::loss masked_cross_entropy [2,4,1024,128256] bf16: forward (one read) + backward to f32 d(logits)")
    del x, tg, mk
    torch.cuda.empty_cache()
    # the generic softmax of the backend at this vocabulary (f32 in, f32 out): a thread-block cluster holds each row in
    # shared memory, so the row crosses HBM once in each direction
    xf = torch.randn(4096, V, generator=gen, device=dev)
    res["lane_softmax_f32"] = entry(4096, _time(lambda: ops.softmax(xf)), 4096 * V * 8, "nrl_lane_op softmax over [4096, 128256] f32 (bytes = the row read once + the result written)")
    res["lane_log_softmax_f32"] = entry(4096, _time(lambda: ops.log_softmax(xf)), 4096 * V * 8, "nrl_lane_op log_softmax over [4096, 128256] f32")
    del xf
    torch.cuda.empty_cache()

    # the step before the path fused into it: logits = hidden · W on the tensor cores (tcgen05), folded to the row
    # statistics out of tensor memory; against the two-step form (cuBLAS product writing bf16 logits, then nrl_row_fwd)
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            pk = json.load(fh)
        tf_sustained, tf_burst, tf_kind = float(pk["bf16_tflops_sustained"]), float(pk["bf16_tflops"]), "measured"
    except Exception:
        tf_sustained, tf_burst, tf_kind = 1400.0, 1590.0, "fallback"
    rows, d6 = 8192, 4096
    hx = torch.randn(rows, d6, generator=gen, device=dev).to(torch.bfloat16)
    wt = (torch.randn(d6, V, generator=gen, device=dev) * (3.0 / d6 ** 0.5)).to(torch.bfloat16)
    tk = torch.randint(0, V, (rows,), generator=gen, device=dev, dtype=torch.int32)
    ws = torch.empty(capi.lib().nrl_readout_workspace_bytes(rows, V, d6, 0), dtype=torch.uint8, device=dev)
    lg = torch.empty(rows, V, dtype=torch.bfloat16, device=dev)
    def two_step():
        torch.matmul(hx, wt, out=lg)
        return ops.row_forward(lg, tokens=tk)

    # the headline's own operation fused with the product: masked sampling + log-prob + entropy
    am = synth.grammar_masks(rows, V, gen, dev)
    un = synth.uniforms(rows, gen, dev)
    ws2 = torch.empty(capi.lib().nrl_readout_workspace_bytes(rows, V, d6, capi.READOUT_SAMPLE), dtype=torch.uint8, device=dev)

    def two_step_sample():
        torch.matmul(hx, wt, out=lg)
        return ops.row_forward(lg, allow=am, uniforms=un)

    # These run at the power cap: the clock, and with it every figure, drops by about a tenth between the first
    # second and the later ones. The modes are therefore timed in turn, three passes over all of them, and each
    # mode's median is reported: one measured after another would favour whichever came first.
    modes = {"fused": lambda: ops.readout_forward(hx, wt, tokens=tk, workspace=ws),
             "round": lambda: ops.readout_forward(hx, wt, tokens=tk, workspace=ws, round_bf16=True),
             "mm": lambda: torch.matmul(hx, wt, out=lg), "two": two_step,
             "sample": lambda: ops.readout_forward(hx, wt, uniforms=un, allow=am, workspace=ws2), "two_sample": two_step_sample}
    seen = {k: [] for k in modes}
    for _ in range(3):
        for k, f in modes.items():
            seen[k].append(_time(f, iters=4, warm=1))
    med = {k: sorted(v)[1] for k, v in seen.items()}
    t_fused, t_round, t_mm, t_two, t_sample, t_two_sample = med["fused"], med["round"], med["mm"], med["two"], med["sample"], med["two_sample"]
    fl = 2.0 * rows * d6 * V
    fo, f2 = ops.readout_forward(hx, wt, tokens=tk, workspace=ws, round_bf16=True, want_logits=True), None
    f2 = ops.row_forward(fo.logits, tokens=tk)
    res["readout_fused"] = {"what": "nrl_readout_fwd: logits = hidden [8192, 4096] x W [4096, 128256] (bf16, f32 accumulators in tensor memory) folded to log-prob of given tokens + entropy + row "
                                    "statistics without writing the logits; two_step = torch.matmul (cuBLAS, bf16 logits written) + nrl_row_fwd on them",
                            "rows": rows, "d": d6, "V": V, "timing": "modes timed in turn, 3 passes of 4 launches each, median per mode", "ms": t_fused, "ms_round_bf16": t_round, "TFLOPs": fl / t_fused / 1e9, "frac_of_sustained_bf16_peak": fl / t_fused / 1e9 / tf_sustained,
                            "frac_of_burst_bf16_peak": fl / t_fused / 1e9 / tf_burst, "peak_kind": tf_kind, "cublas_product_alone_ms": t_mm, "cublas_TFLOPs": fl / t_mm / 1e9,
                            "two_step_ms": t_two, "speedup_vs_two_step": t_two / t_fused, "rows_per_s": rows / (t_fused * 1e-3),
                            "values_outside_tolerance_vs_row_fwd_on_its_logits": close(fo.logp, f2.logp) + close(fo.entropy, f2.entropy),
                            "masked_sampling": {"what": "the same product with U8 grammar masks and inverse-CDF sampling fused (NRL_READOUT_SAMPLE): tokens + log-probs + entropy; two_step = cuBLAS + nrl_row_fwd "
                                                        "(masked sampling) on the bf16 logits it wrote", "ms": t_sample, "TFLOPs": fl / t_sample / 1e9, "two_step_ms": t_two_sample,
                                                "speedup_vs_two_step": t_two_sample / t_sample, "rows_per_s": rows / (t_sample * 1e-3)}}
    return res


def run_readout_variant(args):
    """Profiling variant: a step is one nrl_readout_fwd launch pair (tcgen05 product + epilogue, then the
    merge) over `--rows` rows (default 8192) of d = 4096 against V = 128256. Not the headline."""
    import torch

    from noetic_tensor_b200 import capi, ops

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    rows, d = args.rows or 8192, 4096
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    hx = torch.randn(rows, d, generator=gen, device=dev).to(torch.bfloat16)
    wt = (torch.randn(d, V, generator=gen, device=dev) * (3.0 / d ** 0.5)).to(torch.bfloat16)
    tk = torch.randint(0, V, (rows,), generator=gen, device=dev, dtype=torch.int32)
    ws = torch.empty(capi.lib().nrl_readout_workspace_bytes(rows, V, d, capi.READOUT_SAMPLE if args.readout_sample else 0), dtype=torch.uint8, device=dev)
    if args.readout_sample:  # masked sampling fused: the tensor-core pass with the mass log, then pick, grouping and draw
        from noetic_tensor_b200 import synth

        am, un = synth.grammar_masks(rows, V, gen, dev), synth.uniforms(rows, gen, dev)
        call = lambda: ops.readout_forward(hx, wt, uniforms=un, allow=am, workspace=ws, one_cta=args.readout_one_cta)
    else:
        call = lambda: ops.readout_forward(hx, wt, tokens=tk, workspace=ws, one_cta=args.readout_one_cta)
    for _ in range(max(1, args.warmup)):
        call()
    torch.cuda.synchronize()
    launches0 = capi.lib().nrl_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        o = call()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            peak, kind = float(json.load(fh)["bf16_tflops_sustained"]), "measured sustained cuBLAS bf16"
    except Exception:
        peak, kind = 1400.0, "fallback"
    tf = 2.0 * rows * d * V / (ms * 1e-3) / 1e12
    print(json.dumps({"metric": "rows/s readout-fused " + ("masked sampling + " if args.readout_sample else "") + "log-prob + entropy, d=4096, V=128256 bf16 (profiling variant, not the headline)", "value": rows / (ms * 1e-3), "unit": "rows/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "dtype": "bf16 operands, f32 accumulators",
                      "config": {"workload": f"hidden [{rows}, {d}] x W [{d}, {V}] -> row statistics"}, "gpu_launches": int(capi.lib().nrl_launch_count() - launches0),
                      "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "peak_kind": kind, "kernel": "readout_fwd_kernel<false>" if (args.readout_one_cta or rows <= 128) else "readout_fwd_pair_kernel<false>", "traffic": None},
                      "refused_rows": int((o.status != 0).sum().item())}))


def run_gumbel_variant(args):
    """Profiling variant: a step is one nrl_sample_gumbel launch (the reference's own Gumbel-max sampler on
    the device) over `--rows` headline-shaped rows (default 4096). Not the headline."""
    import torch

    from noetic_tensor_b200 import capi, ops, synth

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    rows = args.rows or 4096
    gen = torch.Generator(device=dev)
    gen.manual_seed(6)
    x = synth.normal_logits(rows, V, 3.0, torch.bfloat16, gen, dev)
    m = synth.grammar_masks(rows, V, gen, dev)
    seed = bytes(range(32))
    for _ in range(max(1, args.warmup)):
        ops.sample_gumbel(x, seed, allow=m)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        ops.sample_gumbel(x, seed, allow=m)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"metric": "rows/s Gumbel-max sampling with the reference's ChaCha20 noise, V=128256 bf16 (profiling variant, not the headline)", "value": rows / (ms * 1e-3), "unit": "rows/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "config": {"workload": f"[{rows}, {V}] bf16 + U8 grammar masks"}, "gpu_launches": args.steps}))


def run_ours(args):
    if args.variant == "readout":
        return run_readout_variant(args)
    if args.variant == "gumbel":
        return run_gumbel_variant(args)
    # stdout carries the one JSON line and nothing else: libraries that write to it (NCCL prints
    # its version there when the communicator comes up) are sent to stderr until the line is printed
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    import torch
    import torch.distributed as dist

    from noetic_tensor_b200 import capi, ops
    from noetic_tensor_b200.hostpath import HostForward

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    capi.lib()
    l2_fetch = None
    if args.l2_fetch_granularity:
        # cudaLimitMaxL2FetchGranularity: a hint of this process's context (it ends with the process; nothing
        # about the GPU itself changes). An experiment switch for profiler captures, not part of the headline.
        import ctypes

        rt = ctypes.CDLL("libcudart.so.12")
        torch.zeros(1, device=dev)
        rc = rt.cudaDeviceSetLimit(5, ctypes.c_size_t(args.l2_fetch_granularity))
        now = ctypes.c_size_t(0)
        rt.cudaDeviceGetLimit(ctypes.byref(now), 5)
        l2_fetch = {"asked": args.l2_fetch_granularity, "rc": rc, "now": now.value}

    # resident batch: as many whole seeds of the config as fit, leaving headroom
    free, total = torch.cuda.mem_get_info(dev)
    per_seed = ROWS_PER_SEED * V * BYTES_PER_ELEM
    headroom = 14 << 30
    s_res = int(max(1, min(S_FULL, (free - headroom) // per_seed)))
    if args.seeds:
        s_res = min(s_res, args.seeds)
    rows = s_res * ROWS_PER_SEED
    if args.rows:
        rows = min(rows, args.rows)  # a small case for profiler captures
    logits, ref, mask, u = make_inputs(rows, 1000 + rank, dev)
    torch.cuda.synchronize()

    if args.variant == "unmasked":  # a profiling variant: the same logits and reference without the mask
        mask = None
    if args.variant in ("backward", "bitmask") and not (args.no_e2e and args.no_extras):
        raise SystemExit(f"--variant {args.variant} is a profiling variant: run it with --no-e2e --no-extras")

    def step():
        return ops.row_forward(logits, ref_logits=ref, allow=mask, uniforms=u)

    if args.variant == "bitmask":  # a profiling variant: the same rows with the mask bit-packed, read by the kernel as it is
        import numpy as np

        bits = torch.cat([torch.from_numpy(np.packbits(mask[a:a + 4096].cpu().numpy(), axis=1, bitorder="little").view(np.int32)) for a in range(0, rows, 4096)]).to(dev)

        def step():
            return ops.row_forward(logits, ref_logits=ref, allow_bits=bits, uniforms=u)

    if args.variant == "backward":  # a profiling variant: the step is one row_bwd launch over the resident rows
        saved = step()
        ones = torch.ones(rows, dtype=torch.float32, device=dev)
        dbuf = torch.empty(rows, V, dtype=torch.float32, device=dev)
        forward_step = step

        def step():
            ops.row_backward(logits, saved, ref_logits=ref, allow=mask, g_logp=ones, g_kl=ones, g_ent=ones, out=dbuf)
            return saved

    sampler = ClockSampler(local)
    sampler.start()  # before the warm-up: nvidia-smi is up and printing by the time the timed region starts
    for _ in range(max(3, args.warmup)):
        out = step()
    torch.cuda.synchronize()
    bad = int((out.status != 0).sum().item())
    sampler.wait_first()

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.begin()
    launches0 = capi.lib().nrl_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = step()
    e1.record()
    torch.cuda.synchronize()
    sampler.end()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    launches = capi.lib().nrl_launch_count() - launches0
    clocks = sampler.stop()
    if not clocks.get("samples"):
        # K steps can be shorter than the sampler's 100 ms period: the same step repeated for ~0.7 s right
        # after the timed region (not timed, not counted) gives the clocks under this load
        probe = ClockSampler(local)
        probe.start()
        probe.wait_first()
        probe.begin()
        t_end = time.perf_counter() + 0.7
        while time.perf_counter() < t_end:
            step()
            torch.cuda.synchronize()
        probe.end()
        clocks = probe.stop()
        clocks["from"] = "the same step repeated for 0.7 s right after the timed region, which was shorter than the sampler's period"
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    ms_per_step = ms_max / args.steps
    value = world * rows / (ms_per_step * 1e-3)

    # bitwise reproducibility of the step, checked outside the timed region
    again = step()
    torch.cuda.synchronize()
    reproducible = bool(torch.equal(out.tokens, again.tokens) and torch.equal(out.logp.view(torch.int32), again.logp.view(torch.int32))
                        and torch.equal(out.kl.view(torch.int32), again.kl.view(torch.int32)) and torch.equal(out.entropy.view(torch.int32), again.entropy.view(torch.int32)))

    # roofline of the one kernel a step launches (this rank's own launch time)
    peak, peak_kind = measured_peak()
    alg_bytes = rows * V * (BYTES_PER_ELEM if mask is not None else 4)
    if args.variant == "bitmask":
        alg_bytes = rows * V * 4 + rows * (V // 8)
    if args.variant == "backward":
        alg_bytes += rows * V * 4  # the forward's reads again + f32 d(logits) written
    launch_ms = ms / args.steps
    achieved = alg_bytes / (launch_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind + " copy bandwidth",
                "frac_of_nominal_8TBs": achieved / 8000.0, "kernel": "row_bwd_kernel<bf16, ref, allow>" if args.variant == "backward" else "nrl_bits::row_fwd_grouped<bf16, ref, allow>" if args.variant == "bitmask" else "row_fwd_grouped<bf16, ref, allow>" if mask is not None else "row_fwd_grouped<bf16, ref, no mask>", "algorithmic_bytes_per_launch": alg_bytes,
                "traffic": None if args.variant in ("backward", "bitmask") else (NCU_TRAFFIC_RATIO if mask is not None else 1.0) * alg_bytes,
                "note": "algorithmic bytes count every logit, reference and mask byte once (5 B per element); the kernel does not read logits the mask "
                        "excludes, so its DRAM traffic (`traffic`, from ncu) is below the algorithmic bytes and `frac` can exceed 1"}
    if roofline["traffic"]:
        roofline["dram_GBps"] = roofline["traffic"] / (launch_ms * 1e-3) / 1e9
        roofline["dram_frac"] = roofline["dram_GBps"] / peak
    if mask is not None and args.variant == "headline":
        # What the masks make necessary: a launch cannot move less than the mask plus the aligned granules of
        # logits and reference that hold an allowed token. `frac` is stated on the 32-byte sector (the unit
        # the memory system addresses); the coarser granules are given beside it.
        nec = {g: necessary_bytes(mask, g) for g in (32, 64, 128)}
        roofline["frac_algorithmic"] = roofline["frac"]
        roofline["necessary_bytes_per_launch"] = nec[128]
        roofline["necessary_bytes_per_launch_64B_granules"] = nec[64]
        roofline["necessary_bytes_per_launch_32B_sectors"] = nec[32]
        roofline["necessary_bytes_per_row"] = nec[128] / rows
        roofline["achieved_necessary"] = nec[128] / (launch_ms * 1e-3) / 1e9
        roofline["frac"] = roofline["achieved_necessary"] / peak
        roofline["frac_32B_sectors"] = nec[32] / (launch_ms * 1e-3) / 1e9 / peak
        roofline["note"] = ("`frac` = necessary bytes ÷ launch time ÷ peak. Necessary bytes: the byte mask whole plus every aligned 128-byte granule of logits and of reference that "
                            "holds an allowed token, counted on the device from the masks of this run. 128 bytes is what this GPU's DRAM moves for an isolated 16-byte load: ncu counts "
                            "1.05x these bytes for the launch, the same with cudaLimitMaxL2FetchGranularity at 32, 64 and 128 (profiles/row_fwd_grouped_sector_counters_4096rows.md); on "
                            "32-byte sectors the figure would be `frac_32B_sectors`. `achieved` / `frac_algorithmic` count every logit, reference and mask byte once (5 B per element) "
                            "although the kernel never reads logits the mask excludes; `traffic` is the DRAM traffic ncu measured on a 4096-row capture scaled by rows")

    # Strong scaling (the partition the path is meant for): ONE config-3 batch split along S, then B, over the
    # ranks, no collective on the data path; and the TokenReduction that spans ranks, run over NCCL and held to
    # the bits of the one-GPU kernel.
    strong = None
    if args.variant == "headline" and not args.no_strong and rows % T == 0:
        from noetic_tensor_b200 import shard

        S_j, B_j = (rows // ROWS_PER_SEED, B) if rows % ROWS_PER_SEED == 0 else (1, rows // T)
        r0, r1 = shard.row_range(S_j, B_j, T, rank, world)
        lg, rf, mk, uu = logits[r0:r1], ref[r0:r1], mask[r0:r1], u[r0:r1]

        def sstep():
            return ops.row_forward(lg, ref_logits=rf, allow=mk, uniforms=uu)

        for _ in range(3):
            so = sstep()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            so = sstep()
        s1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        tmax = torch.tensor([s0.elapsed_time(s1) / args.steps], device=dev, dtype=torch.float64)
        tmin = tmax.clone()
        if world > 1:
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
        per_local = so.logp.reshape(-1, T).contiguous()
        full = shard.gather_sequences(per_local, S_j, B_j).reshape(S_j, B_j, T).contiguous()
        bitwise = True
        for red in (capi.REDUCE_SUM, capi.REDUCE_TOKEN_MEAN, capi.REDUCE_PER_SEQUENCE, capi.REDUCE_SEQUENCE_MEAN):
            sharded = shard.ShardedReduction(per_local, None, red, S_j, B_j).value
            whole = ops.reduce_tokens(full, None, red)
            bitwise = bitwise and bool(torch.equal(sharded.view(torch.int32), whole.view(torch.int32)))
        flag = torch.tensor([1 if bitwise else 0], device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        total_rows = S_j * B_j * T
        strong = {"scaling": "strong", "rows_total_per_step": total_rows, "rows_this_rank": r1 - r0, "ms_per_step": float(tmax.item()), "ms_per_step_fastest_rank": float(tmin.item()),
                  "value": total_rows / (float(tmax.item()) * 1e-3), "unit": "rows/s", "sharded_reduce_bitwise": bool(flag.item()),
                  "note": f"one config-3 batch of {S_j} seed(s) split along S then B over {world} rank(s) (shard.row_range), each rank one launch over its rows, max over ranks; "
                          "no collective on the data path. The cross-rank TokenReduction (nrl_reduce_tokens_partial -> all_gather of two floats per sequence over NCCL -> "
                          "nrl_reduce_tokens_fold) is compared, outside the timed region, with nrl_reduce_tokens on the gathered per-token values: same bits for Sum, TokenMean, "
                          "PerSequence, SequenceMean"}

    # end to end from host memory: pinned inputs cross PCIe every step, results come back
    e2e = None
    if not args.no_e2e:
        e2e_rows = min(args.e2e_rows, rows)
        from noetic_tensor_b200.hostpath import bind_host_thread_near

        near = bind_host_thread_near(dev)  # the pinned buffers below land in the memory next to this rank's GPU
        hf = HostForward(V, torch.bfloat16, chunk_rows=512, device=dev)
        if mask is None:
            raise SystemExit("--variant unmasked is a profiling variant: run it with --no-e2e")
        hx, hr, hm, hu = (t_[:e2e_rows].cpu().pin_memory() for t_ in (logits, ref, mask, u))
        hf.run(hx, hu, ref=hr, mask=hm)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e2e_steps = 3
        for _ in range(e2e_steps):
            hout = hf.run(hx, hu, ref=hr, mask=hm)
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        te = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        cmp_packed = compare_with_resident(hout, out, e2e_rows)
        packed_rate = world * e2e_rows / float(te.item())
        packed_bytes, packed_live = hf.h2d_bytes, hf.live_vectors
        # the same rows read in place: pinned host memory is mapped into the device's address space
        hf.run_mapped(hx, hu, ref=hr, mask=hm, first_chunk_rows=512)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            mout = hf.run_mapped(hx, hu, ref=hr, mask=hm, first_chunk_rows=512)
        tm = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        mapped_rate = world * e2e_rows / float(tm.item())
        cmp_mapped = compare_with_resident(mout, out, e2e_rows)
        # the same byte mask turned into bits by host threads inside the timed region: V/8 mask bytes per row cross the link
        hf.run_mapped(hx, hu, ref=hr, mask=hm, chunk_rows=1184, first_chunk_rows=512, pack_bits_on_host=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            pout = hf.run_mapped(hx, hu, ref=hr, mask=hm, chunk_rows=1184, first_chunk_rows=512, pack_bits_on_host=True)
        tp = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tp, op=dist.ReduceOp.MAX)
        hostbits_rate = world * e2e_rows / float(tp.item())
        hostbits_ok = bool((pout["tokens"] == mout["tokens"]).all())
        cmp_hostbits = compare_with_resident(pout, out, e2e_rows)
        # both at once on two shares of the rows: the mapped path is bound by the small reads the link keeps in flight,
        # the packed path by the host's cores and memory
        hf.run_hybrid(hx, hu, ref=hr, mask=hm)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            yout = hf.run_hybrid(hx, hu, ref=hr, mask=hm)
        ty = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ty, op=dist.ReduceOp.MAX)
        hybrid_rate = world * e2e_rows / float(ty.item())
        cmp_hybrid = compare_with_resident(yout, out, e2e_rows)
        hybrid_packed_rows = int(e2e_rows * 0.375) // 512 * 512
        # a caller that holds bit-packed masks (what grammar engines emit): V/8 mask bytes per row go up
        import numpy as np
        hbits = torch.from_numpy(np.packbits(hm.numpy(), axis=1, bitorder="little").view(np.int32)).pin_memory()
        hf.run_mapped(hx, hu, ref=hr, mask_bits=hbits, first_chunk_rows=512)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            bout = hf.run_mapped(hx, hu, ref=hr, mask_bits=hbits, first_chunk_rows=512)
        bits_rate = e2e_rows / ((time.perf_counter() - t0) / e2e_steps)
        bits_ok = bool((bout["tokens"] == mout["tokens"]).all())
        cmp_bits = compare_with_resident(bout, out, e2e_rows)
        # what the host link gives every rank at once for plain copies of whole rows: the ceiling of an upload that
        # does not use the mask, and the yardstick for the bytes the modes above move
        scratch = torch.empty_like(hx, device=dev)
        scratch.copy_(hx, non_blocking=True)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            scratch.copy_(hx, non_blocking=True)
        torch.cuda.synchronize()
        tc = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tc, op=dist.ReduceOp.MAX)
        copy_gbps = world * hx.numel() * hx.element_size() / float(tc.item()) / 1e9
        del scratch
        all_cmp = {"packed": cmp_packed, "mapped": cmp_mapped, "mapped_host_bits": cmp_hostbits, "hybrid": cmp_hybrid, "bit_packed_masks": cmp_bits}
        e2e_matches = all(c["values_outside_tolerance"] == 0 and c["tokens_differing"] <= max(1, e2e_rows // 1000) for c in all_cmp.values())
        h2d, d2h = hf.bytes_per_row()
        mapped_bytes = e2e_rows * (V + 4) + packed_live * 8 * 2 * 2  # the mask whole and the uniforms + the live vectors of bf16 logits and reference
        hostbits_bytes = mapped_bytes - e2e_rows * V + e2e_rows * (V // 8)
        hybrid_bytes = hostbits_bytes * (e2e_rows - hybrid_packed_rows) / e2e_rows + packed_bytes * hybrid_packed_rows / e2e_rows
        modes = {"mapped": (mapped_rate, mapped_bytes), "packed": (packed_rate, packed_bytes), "mapped, mask bit-packed on the host": (hostbits_rate, hostbits_bytes),
                 "hybrid: 5/8 of the rows mapped with host-packed bit masks, 3/8 packed by host threads, at the same time": (hybrid_rate, hybrid_bytes)}
        best = max(modes, key=lambda k: modes[k][0])
        e2e = {"value": modes[best][0], "unit": "rows/s", "mode": best,
               "h2d_bytes_per_step": int(modes[best][1]), "d2h_bytes_per_step": e2e_rows * d2h,
               "host_bytes_per_step": e2e_rows * h2d, "rows_per_step": e2e_rows, "host_cpus_near_gpu": (len(near) if near else None), "matches_resident_path": e2e_matches, "vs_resident_path": all_cmp,
               "host_link": {"h2d_copy_GBps_all_ranks": copy_gbps, "whole_rows_per_s_at_that_rate": copy_gbps * 1e9 / (V * BYTES_PER_ELEM),
                             "moved_GBps_estimate": modes[best][1] / e2e_rows * modes[best][0] / 1e9,
                             "note": "every rank copies its pinned bf16 logits (2.1 GB) to its GPU at the same time, max over ranks: what uploading whole rows (logits + reference + mask, 5 B per "
                                     "element) could reach at best, beside what the fastest mode moves by the estimate of h2d_bytes_per_step"},
               "h2d_bytes_note": "for the mapped modes an estimate: the mask bytes that are copied plus 16 B per live vector per stream; the link moves at least a 32-byte sector per isolated vector and has no counter here",
               "mapped": {"value": mapped_rate, "h2d_bytes_per_step_estimate": int(mapped_bytes),
                          "note": "nrl_row_fwd is given the pinned host logits and reference themselves (mapped into the device's address space) and fetches only the vectors the mask allows "
                                  "over the host link; the byte mask, read whole, goes up by copies in 2048-row chunks (the first one 512 rows) one chunk ahead of the kernel; uniforms go up and per-row results come back by copies, all inside the timed region; "
                                  "the byte count is an estimate (mask bytes + live vectors), the link has no counter here"},
               "mapped_host_bits": {"value": hostbits_rate, "h2d_bytes_per_step_estimate": int(hostbits_bytes), "host_threads": hf.threads, "same_tokens_as_mapped": hostbits_ok,
                                    "note": "as `mapped` with 1184-row chunks, but host threads turn each chunk's byte mask into one bit per token (nrl_host_pack_bits, inside the timed region, one chunk ahead of the kernel) "
                                            "and the kernels read the bits (NRL_FWD_MASK_BITS): the mask crosses the link as V/8 bytes per row; results are the byte mask's bit for bit"},
               "bit_packed_masks": {"value": bits_rate, "this_rank_only": True, "same_tokens": bits_ok, "h2d_bytes_per_step_estimate": int(mapped_bytes - e2e_rows * V + e2e_rows * (V // 8)),
                                    "note": "not the headline input format: the same rows from a caller that holds int32 bit masks [rows, V/32], which the kernels read as they are (NRL_FWD_MASK_BITS)"},
               "hybrid": {"value": hybrid_rate, "h2d_bytes_per_step_estimate": int(hybrid_bytes), "rows_packed": hybrid_packed_rows, "host_threads": hf.threads,
                          "note": "HostForward.run_hybrid: two shares of the rows at the same time on two Python threads and two CUDA streams, the first through the mapped path with host-packed bit masks, "
                                  "the last 3/8 through the packed path (half of the host threads each); every row by the same kernels as in those modes"},
               "packed": {"value": packed_rate, "h2d_bytes_per_step": int(packed_bytes), "packed_chunks": hf.packed_chunks, "whole_chunks": hf.whole_chunks, "host_threads": hf.threads,
                          "note": "512-row chunks, double-buffered: host threads keep the vectors the mask allows (nrl_host_pack), those cross PCIe by copies, a kernel puts them in place "
                                  "(nrl_unpack_rows), then the same forward; the packing runs inside the timed region"},
               "note": "host-resident bf16 logits + reference + U8 mask in pinned memory (host_bytes_per_step) through the C ABI, results back in pinned host memory; "
                       "value is the fastest of the host paths, named in `mode`"}

    extras = None
    if rank == 0 and not args.no_extras:
        del logits, ref, mask, u, out, again
        torch.cuda.empty_cache()
        extras = run_extras(dev, peak)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        n = 24
        xb, rb, al = host_sample(n, 1234)
        cpu_reference_rows(xb[:2], rb[:2], al[:2], 1, False, 1)
        dt = cpu_reference_rows(xb, rb, al, 2, False, 1)
        cpu_baseline = {"value": n / dt, "unit": "rows/s", "cores": 1, "kind": "port",
                        "sample": f"{n} rows of the workload; C++ restatement of the reference's Cpu(Reference) op sequence (sample_categorical Gumbel-max + "
                                  "token_log_probs + reference_kl + categorical_entropy), single thread as Cpu(Reference) is"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config 3 [8,32,1024,128256] bf16 + U8 grammar mask + bf16 reference stream (headline)" if args.variant == "headline" else "config 3 rows, the d(logits) kernel alone (profiling variant, not the headline)" if args.variant == "backward" else "config 3 rows with the mask bit-packed (profiling variant, not the headline)" if args.variant == "bitmask" else "config 3 logits + reference WITHOUT the mask (profiling variant, not the headline)",
                       "storage": "bf16 logits, f32 arithmetic", "S_resident_per_gpu": s_res, "B": B, "T": T, "V": V,
                       "rows_per_gpu_per_step": rows, "cache": "inputs (tens of GB) far larger than the 126 MB L2; no flush needed", "partition": f"rows split across {world} rank(s), no collective"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "bitwise_reproducible": reproducible, "refused_rows": bad, "strong_scaling": strong, "l2_fetch_granularity": l2_fetch,
            "samplers": {"ours": "inverse CDF against one caller-supplied uniform per row, fused into the forward (what the path is defined on)",
                         "reference_arm": "the reference's Gumbel-max (one ChaCha20 u64 and two f64 logarithms per logit) on the host cores",
                         "same_algorithm_on_device": None if not extras else {"rows_per_s": extras["reference_gumbel_sampler"]["rows_per_s"],
                                                                              "vs_cpu_baseline_1_core": (extras["reference_gumbel_sampler"]["rows_per_s"] / cpu_baseline["value"]) if cpu_baseline else None,
                                                                              "what": "nrl_sample_gumbel: the reference's own sampler, token for token, on the device (extras.reference_gumbel_sampler)"}},
            "extras": extras,
        }
        sys.stdout.flush()
        os.dup2(json_fd, 1)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seeds", type=int, default=0, help="cap the resident seeds per GPU (default: as many of the 8 as fit)")
    ap.add_argument("--e2e-rows", type=int, default=8192)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--variant", default="headline", choices=["headline", "unmasked", "backward", "bitmask", "readout", "gumbel"],
                    help="unmasked: drop the mask (for profiling the every-byte-read path); backward: time the d(logits) kernel alone; bitmask: the mask bit-packed; none of them is the headline")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary measurements (backward, PPO step, other configs)")
    ap.add_argument("--l2-fetch-granularity", type=int, default=0, help="set cudaLimitMaxL2FetchGranularity (32, 64, 128) for this process: an experiment switch for profiler captures")
    ap.add_argument("--readout-one-cta", action="store_true", help="--variant readout: one CTA per 128 rows (NRL_READOUT_ONE_CTA) instead of CTA pairs")
    ap.add_argument("--readout-sample", action="store_true", help="--variant readout: U8 grammar masks and inverse-CDF sampling fused (NRL_READOUT_SAMPLE) instead of given tokens")
    ap.add_argument("--no-strong", action="store_true", help="skip the strong-scaling measurement and the cross-rank TokenReduction check")
    ap.add_argument("--rows", type=int, default=0, help="cap the resident rows per GPU (small cases for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
