"""Benchmark of the QLoRA hot path on B200: fused LM-head + cross-entropy forward+backward.

    python bench.py --gpus N --steps K --warmup W            # this repository's kernels
    python bench.py --impl reference --gpus N --steps K --warmup W   # the CPU restatement, timed

One "step" is one pass of the hot path over one batch of synthetic input: fused_head_loss forward
plus backward through the public API (loss, per-row loss/entropy/accuracy, dHidden). The workload
at N=1 is benchmark config 1 (2048 packed tokens, hidden 1536, tied fp16 head 151936 x 1536, 10 %
ignored targets). At N>1 the head is vocabulary-parallel with 2048 tokens per GPU (weak scaling:
per-GPU GEMM work is constant, the exchange is one all-gather of the per-row states and one
all-reduce of dHidden). `--workload c5a` selects the fixed 65536-token job instead.

The printed line carries: `value` (tokens/s, inputs resident in HBM), `e2e` (the same through host
buffers: pinned host -> device copies of hidden and targets and device -> host reads of the loss
and dHidden inside the timed region), `roofline` (tensor-pipe bound, measured per kernel class with
CUDA events on the launching stream), `kernels` (the memory-bound kernels of the path in GB/s
against the measured HBM copy peak, cold L2 by rotating buffer sets) and `cpu_baseline` (the oracle
on the host cores over a bounded sample of the same workload).
"""

import argparse
import ctypes
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, VOCAB, TOKENS_PER_GPU = 1536, 151936, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:  # noqa: BLE001
        return dict(FALLBACK_PEAKS), "fallback"


SLAB = 2048   # rows of hidden states generated from one seed


def make_weight():
    """The tied head weight of benchmark config 1: [151936, 1536] ~N(0, 0.02) fp16, generated on the
    CPU slab by slab (no 900 MB fp32 temporary) so that oracle and kernels see identical bits."""
    gen = torch.Generator().manual_seed(1000)
    weight = torch.empty(VOCAB, HIDDEN, dtype=torch.float16)
    for r0 in range(0, VOCAB, 16384):
        rows = min(16384, VOCAB - r0)
        weight[r0:r0 + rows] = (torch.randn(rows, HIDDEN, generator=gen) * 0.02).half()
    return weight


def make_rows(slab):
    """Slab `slab` of the token rows: hidden [2048, 1536] ~N(0,1) fp16 and targets uniform over the
    vocabulary with 10 % set to ignore_index (benchmark config 1 recipe). Every slab has its own
    seed, so a rank generates only the rows it feeds and any rank can regenerate any row."""
    gen = torch.Generator().manual_seed(2000 + slab)
    hidden = torch.randn(SLAB, HIDDEN, generator=gen).half()
    target = torch.randint(0, VOCAB, (SLAB,), generator=gen)
    target[torch.rand(SLAB, generator=gen) < 0.1] = -100
    return hidden, target


def make_local_rows(rank, slabs_per_rank):
    parts = [make_rows(rank * slabs_per_rank + i) for i in range(slabs_per_rank)]
    return torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts])


def make_inputs(n_tokens):
    """Config 1 inputs for a single process: (hidden, weight, target) of n_tokens rows."""
    hidden, target = make_local_rows(0, -(-n_tokens // SLAB))
    return hidden[:n_tokens].contiguous(), make_weight(), target[:n_tokens].contiguous()


class ClockSampler:
    """Reads SM clocks and clock-event reasons through NVML from a thread of this process while
    the timed regions run (read-only queries, 10 ms apart). An nvidia-smi child process polling at
    that rate was seen to stall kernel launches for milliseconds, which is why it is not used."""

    PERIOD_S = 0.010

    def __init__(self, index):
        self.samples, self.index = [], index
        self.windows = []   # (start, end) wall-clock spans of the timed regions
        self.handle = self.thread = self.nvml = None
        self.stop = threading.Event()
        self.max_mhz = None

    def __enter__(self):
        if os.environ.get("SOUP_BENCH_NO_CLOCKS"):   # measurement-hygiene experiments only
            return self
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.index
            if visible:  # NVML numbers the physical devices
                entries = [v for v in visible.split(",") if v.strip() != ""]
                if index < len(entries) and entries[index].strip().isdigit():
                    index = int(entries[index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001
            self.handle = None
        return self

    def wait_first_sample(self, limit_s=2.0):
        t0 = time.time()
        while self.handle is not None and not self.samples and time.time() - t0 < limit_s:
            time.sleep(0.01)

    def _poll(self):
        nv = self.nvml
        while not self.stop.is_set():
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                self.samples.append((mhz, reasons, time.time()))
            except Exception:  # noqa: BLE001
                break
            self.stop.wait(self.PERIOD_S)

    def __exit__(self, *exc):
        self.stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def window_mhz(self, index):
        """Median SM clock of the samples that fell inside timed region `index` (None if none)."""
        if index >= len(self.windows):
            return None
        a, b = self.windows[index]
        inside = [s[0] for s in self.samples if a <= s[2] <= b]
        return statistics.median(inside) if inside else None

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        nv = self.nvml
        inside = [s for s in self.samples if any(a <= s[2] <= b for a, b in self.windows)]
        used = inside or self.samples
        names = (("hw_slowdown", nv.nvmlClocksEventReasonHwSlowdown),
                 ("hw_thermal_slowdown", nv.nvmlClocksEventReasonHwThermalSlowdown),
                 ("sw_thermal_slowdown", nv.nvmlClocksEventReasonSwThermalSlowdown),
                 ("sw_power_cap", nv.nvmlClocksEventReasonSwPowerCap))
        reasons = [n for n, bit in names if any(s[1] & bit for s in used)]
        sm = [s[0] for s in used]
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(used),
                "scope": "inside the timed regions" if inside else "whole run (no sample fell inside a region)"}


def cpu_head_tokens_per_s(hidden, weight, target, rows, threads):
    """The oracle (fp32 matmul + log_softmax + autograd) over `rows` rows of the workload."""
    from oracle.head_ce import head_ce

    torch.set_num_threads(threads)
    t0 = time.perf_counter()
    head_ce(hidden[:rows], weight, target[:rows])
    return rows / (time.perf_counter() - t0)


def run_reference(args, rank):
    """--impl reference: the CPU restatement of the reference's arithmetic on the host cores."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    hidden, weight, target = make_inputs(TOKENS_PER_GPU)
    w32 = weight.float()
    probe = cpu_head_tokens_per_s(hidden, w32, target, 32, cores)
    budget = 150.0 / max(1, args.steps + args.warmup)  # seconds per step
    rows = int(max(32, min(TOKENS_PER_GPU, probe * budget * 0.8)) // 32 * 32)
    for _ in range(args.warmup):
        cpu_head_tokens_per_s(hidden, w32, target, rows, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_head_tokens_per_s(hidden, w32, target, rows, cores)
    dt = time.perf_counter() - t0
    value = rows * args.steps / dt
    line = {
        "impl": "reference", "metric": "fused LM-head+CE fwd+bwd tokens/s", "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[0]: fused LM-head+CE fwd+bwd, H=1536 V=151936, "
                               f"{rows}-row sample of the 2048-token batch per step"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{rows} rows x full vocabulary per step, torch fp32 matmul + "
                                   "log_softmax + autograd (oracle/head_ce.py)"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# memory-bound kernels of the path, cold L2 (rotating buffer sets larger than the 126 MB L2)
# ------------------------------------------------------------------------------------------
PLAIN_LAUNCHES = False   # --plain-launches: no graphs, a few direct launches per case (for ncu)


def time_rotating(make_call, n_sets, reps=10):
    """Milliseconds per call of `make_call(i)`: the calls over all n_sets buffer sets are captured
    into one CUDA graph (so the host's launch cost is out of the picture and consecutive launches
    touch different, L2-cold buffers) and the graph is replayed `reps` times between two events."""
    if PLAIN_LAUNCHES:
        n = min(n_sets, 3)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            make_call(i)
        b.record()
        b.synchronize()
        return a.elapsed_time(b) / n
    for i in range(n_sets):
        make_call(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(n_sets):
            make_call(i)
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / (reps * n_sets)


def kernel_suite(dev, hbm_peak, n_rows=2048, tag="", with_nf4=True):
    from claudemaxing_b200 import _lib, lora, qlora
    from claudemaxing_b200.nf4 import dequantize_nf4
    from claudemaxing_b200.swiglu_recompute import _silu_mul_bwd, _silu_mul_fwd

    out = {}
    f16, f32 = torch.float16, torch.float32

    def sets_for(nbytes):
        return max(2, int(400e6 // max(nbytes, 1)) + 1)

    def record(name, ms, nbytes, launches=1):
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name + tag] = {"ms": round(ms, 5), "gb_s": round(gbs, 1), "frac_of_measured_hbm": round(gbs / hbm_peak, 3),
                     "frac_of_nominal_8000": round(gbs / 8000.0, 3),
                     "algorithmic_bytes": int(nbytes), "launches": launches}

    if with_nf4:
        # Context for the write-heavy kernels: what torch's own copy and fill reach on this GPU,
        # timed the same way (NF4 dequant writes four bytes for every byte it reads).
        big_a = [torch.empty(256 << 20, dtype=torch.uint8, device=dev) for _ in range(3)]
        ms = time_rotating(lambda i: big_a[(i + 1) % 3].copy_(big_a[i]), 3)
        record("reference_torch_copy_256MiB", ms, 2 * (256 << 20))
        ms = time_rotating(lambda i: big_a[i].zero_(), 3)
        record("reference_torch_fill_256MiB", ms, 256 << 20)
        del big_a
        # NF4 dequant: the seven projection shapes of one Qwen2.5-1.5B layer, 28 distinct layers
        shapes = [(1536, 1536), (256, 1536), (256, 1536), (1536, 1536), (8960, 1536), (8960, 1536),
                  (1536, 8960)]
        code, code2 = qlora.normal_float4_levels().to(dev), qlora.absmax_levels().to(dev)
        layers = []
        gen = torch.Generator(device=dev).manual_seed(1)
        for _ in range(28):
            layer = []
            for (o, i) in shapes:
                n = o * i
                packed = torch.randint(0, 256, (n // 2, 1), dtype=torch.uint8, device=dev, generator=gen)
                absmax8 = torch.randint(0, 256, (n // 64,), dtype=torch.uint8, device=dev, generator=gen)
                inner = qlora.QuantState(torch.rand(-(-n // 64 // 256), device=dev, generator=gen) * 0.01,
                                         (n // 64,), code2, 256, f32)
                st = qlora.QuantState(absmax8, (o, i), code, 64, f16,
                                      offset=torch.tensor([0.02], device=dev), state2=inner)
                layer.append((packed, st))
            layers.append(layer)
        outs = [torch.empty(o * i, dtype=f16, device=dev).view(o, i) for (o, i) in shapes]
        elems = sum(o * i for o, i in shapes)

        def nf4_all():
            for layer in layers:
                for (packed, st), buf in zip(layer, outs):
                    dequantize_nf4(packed, st, f16, out=buf)

        ms_all = time_rotating(lambda i: nf4_all(), 1, reps=5)
        record("nf4_dequant_28_layers", ms_all, 2.51587 * elems * 28, launches=28 * 7)
        from claudemaxing_b200.nf4 import dequantize_nf4_batch

        def nf4_all_batched():  # the seven projections of a layer in one launch
            for layer in layers:
                dequantize_nf4_batch(layer, f16, outs=outs)

        ms_b = time_rotating(lambda i: nf4_all_batched(), 1, reps=5)
        record("nf4_dequant_28_layers_batched_per_layer", ms_b, 2.51587 * elems * 28, launches=28)
        big = [(l[4][0], l[4][1]) for l in layers]  # the 8960 x 1536 gate projections, one per layer
        ms = time_rotating(lambda i: dequantize_nf4(big[i][0], big[i][1], f16, out=outs[4]), len(big))
        record("nf4_dequant_8960x1536", ms, 2.51587 * 8960 * 1536)
        del layers, big

    H, I = 1536, 8960
    # RMSNorm, variant A (fp16 x, fp16 w) and variant B (fp32 x, fp32 w, fp16 copy + side buffer)
    nA = sets_for(3 * n_rows * H * 2)
    xa = [torch.randn(n_rows, H, device=dev, dtype=f16) for _ in range(nA)]
    dya = [torch.randn(n_rows, H, device=dev, dtype=f16) for _ in range(nA)]
    oa = [torch.empty(n_rows, H, device=dev, dtype=f16) for _ in range(nA)]
    wa = (torch.rand(H, device=dev) + 0.5).half()
    rstd = torch.empty(n_rows, device=dev)
    code_f16 = _lib.F16

    def rms_fwd_a(i):
        _lib.call("soup_rmsnorm_fwd", xa[i].data_ptr(), wa.data_ptr(), oa[i].data_ptr(), rstd.data_ptr(),
                  None, None, None, 1, n_rows, H, 1e-6, code_f16, code_f16, code_f16,
                  torch.cuda.current_stream().cuda_stream)

    def rms_bwd_a(i):
        _lib.call("soup_rmsnorm_bwd", dya[i].data_ptr(), xa[i].data_ptr(), wa.data_ptr(), rstd.data_ptr(),
                  oa[i].data_ptr(), None, None, None, None, 1, n_rows, H, code_f16, code_f16,
                  code_f16, code_f16, 0, torch.cuda.current_stream().cuda_stream)

    record("rmsnorm_fwd_f16", time_rotating(rms_fwd_a, nA), 2 * n_rows * H * 2 + 4 * n_rows + 2 * H)
    record("rmsnorm_bwd_f16", time_rotating(rms_bwd_a, nA), 3 * n_rows * H * 2 + 4 * n_rows)
    del xa, dya, oa
    nB = sets_for(10 * n_rows * H)
    xb = [torch.randn(n_rows, H, device=dev) for _ in range(nB)]
    ob = [torch.empty(n_rows, H, device=dev) for _ in range(nB)]
    lb = [torch.empty(n_rows, H, device=dev, dtype=f16) for _ in range(nB)]
    wb = torch.rand(H, device=dev) + 0.5
    tiny = torch.randperm(H, device=dev)[:15]
    wb[tiny] = 5e-4
    slots = torch.full((H,), -1, dtype=torch.int32, device=dev)
    slots[tiny] = torch.arange(15, dtype=torch.int32, device=dev)
    small = torch.empty(n_rows, 15, device=dev, dtype=f16)

    def rms_fwd_b(i):
        _lib.call("soup_rmsnorm_fwd", xb[i].data_ptr(), wb.data_ptr(), ob[i].data_ptr(), rstd.data_ptr(),
                  lb[i].data_ptr(), slots.data_ptr(), small.data_ptr(), 15, n_rows, H, 1e-6, _lib.F32,
                  _lib.F32, _lib.F32, torch.cuda.current_stream().cuda_stream)

    record("rmsnorm_fwd_f32_with_f16_copy", time_rotating(rms_fwd_b, nB), 10 * n_rows * H + 4 * n_rows)

    def rms_bwd_b(i):  # the 4-bit model's backward: fp32 dy, the fp16 copy of the output, fp32 dx
        _lib.call("soup_rmsnorm_bwd", xb[i].data_ptr(), lb[i].data_ptr(), wb.data_ptr(), rstd.data_ptr(),
                  ob[i].data_ptr(), None, None, slots.data_ptr(), small.data_ptr(), 15, n_rows, H,
                  _lib.F32, code_f16, _lib.F32, _lib.F32, 1, torch.cuda.current_stream().cuda_stream)

    record("rmsnorm_bwd_from_f16_copy", time_rotating(rms_bwd_b, nB), 10 * n_rows * H + 4 * n_rows)
    d16 = torch.empty(n_rows, H, device=dev, dtype=f16)

    def rms_bwd_res(i):  # the same with the residual gradient added and the fp16 copy of the sum written
        _lib.call("soup_rmsnorm_bwd_residual", xb[i].data_ptr(), lb[i].data_ptr(), wb.data_ptr(),
                  rstd.data_ptr(), xb[(i + 1) % nB].data_ptr(), ob[i].data_ptr(), d16.data_ptr(),
                  slots.data_ptr(), small.data_ptr(), 15, n_rows, H, torch.cuda.current_stream().cuda_stream)

    record("rmsnorm_bwd_residual_from_f16_copy", time_rotating(rms_bwd_res, nB), 16 * n_rows * H + 4 * n_rows)
    del xb, ob, lb

    # RoPE: packed row [1, n_rows], 12 q heads / 2 kv heads, head_dim 128
    nR = sets_for(2 * 14 * n_rows * 128 * 2)
    lens = [n_rows // 4, n_rows * 3 // 16, n_rows * 5 // 16, n_rows // 4]
    pos = torch.cat([torch.arange(x) for x in lens] + [torch.arange(n_rows - sum(lens))])
    inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, dtype=f32) / 128))
    emb = torch.cat((pos.float()[:, None] * inv,) * 2, -1)[None]
    cos, sin = emb.cos().to(dev, f16), emb.sin().to(dev, f16)
    qs = [torch.randn(1, n_rows, 12 * 128, device=dev, dtype=f16).view(1, n_rows, 12, 128).transpose(1, 2)
          for _ in range(nR)]
    ks = [torch.randn(1, n_rows, 2 * 128, device=dev, dtype=f16).view(1, n_rows, 2, 128).transpose(1, 2)
          for _ in range(nR)]
    rope_bytes = 2 * 14 * n_rows * 128 * 2 + 2 * n_rows * 128 * 2
    qo = [torch.empty(1, 12, n_rows, 128, device=dev, dtype=f16) for _ in range(nR)]
    ko = [torch.empty(1, 2, n_rows, 128, device=dev, dtype=f16) for _ in range(nR)]

    def rope_call(i, backward):
        q, k = qs[i], ks[i]
        _lib.call("soup_rope", q.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                  qo[i].data_ptr(), ko[i].data_ptr(), 1, 12, 2, n_rows, 128, *q.stride()[:3],
                  *k.stride()[:3], 0, cos.stride(1), _lib.F16, _lib.F16, _lib.F16, _lib.F16, _lib.F16,
                  int(backward), torch.cuda.current_stream().cuda_stream)

    record("rope_fwd_q_and_k", time_rotating(lambda i: rope_call(i, False), nR), rope_bytes)
    record("rope_bwd_q_and_k", time_rotating(lambda i: rope_call(i, True), nR), rope_bytes)
    cos32, sin32 = cos.float(), sin.float()
    term = torch.randn(n_rows, 12 * 128, device=dev, dtype=f16).view(1, n_rows, 12, 128).transpose(1, 2)
    qt = [torch.empty(n_rows, 12, 128, device=dev, dtype=f16) for _ in range(nR)]
    kt = [torch.empty(n_rows, 2, 128, device=dev, dtype=f16) for _ in range(nR)]

    def rope_sum_call(i):   # the fused block's form: q + adapter term, fp32 tables, token-major fp16 out
        q, k = qs[i], ks[i]
        qv, kv = qt[i].unsqueeze(0).transpose(1, 2), kt[i].unsqueeze(0).transpose(1, 2)
        _lib.call("soup_rope_sum", q.data_ptr(), term.data_ptr(), k.data_ptr(), cos32.data_ptr(),
                  sin32.data_ptr(), qt[i].data_ptr(), kt[i].data_ptr(), 1, 12, 2, n_rows, 128,
                  *q.stride()[:3], *k.stride()[:3], 0, cos32.stride(1), *term.stride()[:3],
                  *qv.stride()[:3], *kv.stride()[:3], _lib.F16, _lib.F16, _lib.F16, _lib.F32, _lib.F16,
                  _lib.F16, 0, torch.cuda.current_stream().cuda_stream)

    record("rope_sum_fwd_q_plus_term_and_k", time_rotating(rope_sum_call, nR),
           rope_bytes + 12 * n_rows * 128 * 2 + 2 * n_rows * 128 * 2)
    del term, qt, kt
    del qo, ko
    del qs, ks

    # SwiGLU forward and recompute-backward writing over its inputs
    nS = sets_for(3 * n_rows * I * 2)
    gs = [torch.randn(n_rows, I, device=dev, dtype=f16) for _ in range(nS)]
    us = [torch.randn(n_rows, I, device=dev, dtype=f16) for _ in range(nS)]
    ys = [torch.randn(n_rows, I, device=dev, dtype=f16) for _ in range(nS)]
    record("silu_mul_fwd", time_rotating(lambda i: _silu_mul_fwd(gs[i], us[i], ys[i], True), nS),
           3 * n_rows * I * 2)
    record("silu_mul_bwd_inplace", time_rotating(lambda i: _silu_mul_bwd(ys[i], gs[i], us[i], gs[i], us[i], True), nS),
           5 * n_rows * I * 2)
    del gs, us, ys

    # LoRA dropout pack / unpack
    nD = sets_for(12 * n_rows * H)
    xs = [torch.randn(n_rows, H, device=dev) for _ in range(nD)]
    ms_ = [torch.rand(n_rows, H, device=dev) > 0.05 for _ in range(nD)]
    packed_out = [lora._pack(xs[i], ms_[i], 1 / 0.95) for i in range(nD)]
    x16 = [x.half() for x in xs]
    dxs = [torch.empty(n_rows, H, device=dev) for _ in range(nD)]
    xd2 = [torch.empty(n_rows, H, device=dev, dtype=f16) for _ in range(nD)]
    cur = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731

    def pack(i):
        _lib.call("soup_dropout_pack", xs[i].data_ptr(), ms_[i].data_ptr(), packed_out[i][0].data_ptr(),
                  packed_out[i][1].data_ptr(), n_rows * H, 1 / 0.95, _lib.F32, cur())

    def unpack(i):
        _lib.call("soup_dropout_unpack", x16[i].data_ptr(), packed_out[i][1].data_ptr(),
                  packed_out[i][0].data_ptr(), xd2[i].data_ptr(), dxs[i].data_ptr(), n_rows * H,
                  1 / 0.95, _lib.F32, cur())

    record("dropout_pack", time_rotating(pack, nD), n_rows * H * (4 + 1 + 2) + n_rows * H // 8)
    record("dropout_unpack", time_rotating(unpack, nD), n_rows * H * (2 + 2 + 2 + 4) + n_rows * H // 8)
    xd_pair = torch.empty(2, n_rows, H, device=dev, dtype=f16)
    bits_pair = torch.empty(2, n_rows * H // 8, device=dev, dtype=torch.uint8)

    def pack2(i):
        _lib.call("soup_dropout_pack2", xs[i].data_ptr(), ms_[i].data_ptr(), ms_[(i + 1) % nD].data_ptr(),
                  xd_pair[0].data_ptr(), xd_pair[1].data_ptr(), bits_pair[0].data_ptr(),
                  bits_pair[1].data_ptr(), n_rows * H, 1 / 0.95, 1 / 0.95, _lib.F32, cur())

    def unpack2(i):
        _lib.call("soup_dropout_unpack2", x16[i].data_ptr(), bits_pair[0].data_ptr(), bits_pair[1].data_ptr(),
                  packed_out[i][0].data_ptr(), packed_out[(i + 1) % nD][0].data_ptr(),
                  xd_pair[0].data_ptr(), xd_pair[1].data_ptr(), dxs[i].data_ptr(), n_rows * H,
                  1 / 0.95, 1 / 0.95, cur())

    record("dropout_pack_two_adapters", time_rotating(pack2, nD),
           n_rows * H * (4 + 2 * 1 + 2 * 2) + 2 * n_rows * H // 8)
    record("dropout_unpack_two_adapters", time_rotating(unpack2, nD),
           n_rows * H * (2 + 2 * 2 + 2 * 2 + 4) + 2 * n_rows * H // 8)
    del xs, ms_, packed_out, x16, dxs, xd2, xd_pair, bits_pair

    if n_rows <= 4096:
        # metrics from logits that exist anyway (the route for steps that end up building them):
        # one warp per row over [n_rows, 151936] fp16, 622 MB at 2048 rows (larger than L2)
        logit_sets = [torch.randn(n_rows, VOCAB, device=dev, dtype=f16) for _ in range(2)]
        tg = torch.randint(0, VOCAB, (n_rows,), device=dev)
        o_loss, o_ent = torch.empty(n_rows, device=dev), torch.empty(n_rows, device=dev)
        o_hit = torch.empty(n_rows, dtype=torch.int32, device=dev)

        def xent(i):
            _lib.call("soup_xent_rows", logit_sets[i].data_ptr(), tg.data_ptr(), o_loss.data_ptr(),
                      o_ent.data_ptr(), o_hit.data_ptr(), n_rows, VOCAB, VOCAB, _lib.F16, cur())

        record("xent_rows_from_logits", time_rotating(xent, 2), n_rows * VOCAB * 2 + n_rows * 20)
    return out



def attention_suite(dev, tensor_peak):
    """The packed row's attention at the training step's shape (the synthetic batch's four rows
    plus the padding segment: 1280 tokens, 12 query / 2 key heads x 128), forward and backward:
    this library's tcgen05 kernels against torch's variable-length flash attention on the same
    tensors. 28 rotating sets of q, k, v (as in the 28 layers of a step). flops: 4 L^2 D per head
    and segment forward (QK^T and PV, causal half), 10 L^2 D backward (five products)."""
    from torch.nn.attention.varlen import varlen_attn

    from claudemaxing_b200 import _lib
    from claudemaxing_b200.attention import attention_gradients

    lens = [300, 280, 296, 292, 112]
    n, hq, hk, d = sum(lens), 12, 2, 128
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
    scale = d ** -0.5
    gen = torch.Generator(device=dev).manual_seed(6)
    sets = [[torch.randn(n, h, d, device=dev, dtype=torch.float16, generator=gen) for h in (hq, hk, hk, hq)]
            for _ in range(28)]
    outs = [torch.empty(n, hq, d, device=dev, dtype=torch.float16) for _ in range(28)]
    lses = [torch.empty(hq, n, device=dev, dtype=torch.float32) for _ in range(28)]
    causal_pairs = sum(l * l / 2 for l in lens)

    def own_fwd(j):
        q, k, v, _ = sets[j]
        _lib.call("soup_attn_fwd", _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(cu), _lib.ptr(outs[j]),
                  _lib.ptr(lses[j]), n, cu.numel() - 1, hq, hk, d, q.stride(0), k.stride(0), v.stride(0),
                  scale, _lib.stream_of(q))

    def own_bwd(j):
        q, k, v, g = sets[j]
        attention_gradients(q, k, v, outs[j], lses[j], g, cu, scale)

    def lib_fwd(j):
        q, k, v, _ = sets[j]
        varlen_attn(q, k, v, cu, cu, n, n, scale=scale, window_size=(-1, 0))

    rng = torch.empty(2, dtype=torch.uint64, device=dev)

    def lib_bwd(j):
        q, k, v, g = sets[j]
        torch.ops.torch_attn._varlen_attn_backward(g, q, k, v, outs[j], lses[j], cu, cu, n, n, True,
                                                   rng, scale, [-1, 0])

    for j in range(28):
        own_fwd(j)
    out = {}
    for leg, own, lib, products in (("fwd", own_fwd, lib_fwd, 2), ("bwd", own_bwd, lib_bwd, 5)):
        flops = products * 2.0 * causal_pairs * d * hq
        ms_own = time_rotating(own, 28, reps=5)
        ms_lib = time_rotating(lib, 28, reps=5)
        out[f"segment_attention_{leg}@1280tokens"] = {
            "ms": round(ms_own, 5), "tflops": round(flops / (ms_own * 1e-3) / 1e12, 1),
            "frac_of_measured_bf16_peak": round(flops / (ms_own * 1e-3) / 1e12 / tensor_peak, 4),
            "torch_varlen_flash_ms": round(ms_lib, 5), "launches": 1 if leg == "fwd" else 2,
            "note": "latency-bound: ~150 CTAs each walking at most three key tiles; the backward "
                    "launch count includes clearing the fp32 dK / dV buffers" if leg == "bwd" else
                    "latency-bound: ~150 CTAs each walking at most three key tiles (score tiles resident in tensor memory between the two softmax passes)"}
    _lib.check_device_status()
    return out


def nf4_gemm_suite(dev, tensor_peak, rows=1280):
    """The projections of one Qwen2.5-1.5B decoder block at the training step's row count, forward
    and input gradient: the tcgen05 GEMM that dequantises NF4 in its operand prologue against the
    two-step path it replaces (this library's dequant kernel into an fp16 buffer, then cuBLAS
    through torch). Weights rotate over 28 layers' worth of packed bytes (655 MB: cold in L2, as
    in a training step); values are random codes, which cost the same as real ones."""
    from claudemaxing_b200 import qlora
    from claudemaxing_b200.nf4 import dequantize_nf4, nf4_linear, nf4_linear_dx

    f16, f32 = torch.float16, torch.float32
    code, code2 = qlora.normal_float4_levels().to(dev), qlora.absmax_levels().to(dev)
    gen = torch.Generator(device=dev).manual_seed(4)
    layers = 28

    def weight(o, i):
        n = o * i
        packed = torch.randint(0, 256, (n // 2, 1), dtype=torch.uint8, device=dev, generator=gen)
        absmax8 = torch.randint(0, 256, (n // 64,), dtype=torch.uint8, device=dev, generator=gen)
        inner = qlora.QuantState(torch.rand(-(-n // 64 // 256), device=dev, generator=gen) * 0.01,
                                 (n // 64,), code2, 256, f32)
        return packed, qlora.QuantState(absmax8, (o, i), code, 64, f16,
                                        offset=torch.tensor([0.02], device=dev), state2=inner)

    out = {}
    cases = (("q_or_o_1536x1536", [(1536, 1536)]), ("k_or_v_256x1536", [(256, 1536)]),
             ("gate_and_up_2x8960x1536", [(8960, 1536), (8960, 1536)]), ("down_1536x8960", [(1536, 8960)]))
    for name, shapes in cases:
        sets = [[weight(o, i) for (o, i) in shapes] for _ in range(layers)]
        k = shapes[0][1]
        x = torch.randn(rows, k, device=dev, dtype=f16)
        grads = [torch.randn(rows, o, device=dev, dtype=f16) for (o, _) in shapes]
        bufs = [torch.empty(o, i, device=dev, dtype=f16) for (o, i) in shapes]
        flops = 2.0 * rows * sum(o * i for o, i in shapes)

        def two_step_fwd(j):
            for (packed, st), buf in zip(sets[j], bufs):
                torch.nn.functional.linear(x, dequantize_nf4(packed, st, f16, out=buf))

        def two_step_dx(j):
            acc = None
            for (packed, st), buf, g in zip(sets[j], bufs, grads):
                part = torch.matmul(g, dequantize_nf4(packed, st, f16, out=buf))
                acc = part if acc is None else acc + part

        legs = (("fwd", lambda j: nf4_linear(x, sets[j]), two_step_fwd),
                ("dx", lambda j: nf4_linear_dx(grads, sets[j], f16), two_step_dx))
        for leg, fused, two_step in legs:
            ms_f = time_rotating(fused, layers, reps=5)
            ms_t = time_rotating(two_step, layers, reps=5)
            out[f"nf4_linear_{leg}_{name}@{rows}rows"] = {
                "ms": round(ms_f, 5), "tflops": round(flops / (ms_f * 1e-3) / 1e12, 1),
                "frac_of_measured_bf16_burst": round(flops / (ms_f * 1e-3) / 1e12 / tensor_peak, 3),
                "two_step_dequant_plus_cublas_ms": round(ms_t, 5),
                "speedup_over_two_step": round(ms_t / ms_f, 3), "flops": flops}
        del sets
    return out


# ------------------------------------------------------------------------------------------
def cpu_oracle_suite(cores):
    """The oracle's CPU torch implementations of the memory-bound ops at config-3 size (2048 rows),
    one timed call each after one warm-up call, all host cores: what the reference's patches fall
    through to on CPU tensors. Returns {suite key: milliseconds}."""
    from oracle import elementwise as ew
    from oracle import nf4 as onf4

    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(2)
    n, H, inter = 2048, 1536, 8960
    out = {}

    def timed_ms(fn):
        fn()
        t0 = time.perf_counter()
        fn()
        return (time.perf_counter() - t0) * 1e3

    x16 = torch.randn(n, H, generator=gen).half()
    w16 = (torch.rand(H, generator=gen) + 0.5).half()
    dy16 = torch.randn(n, H, generator=gen).half()
    x32, w32, dy32 = x16.float(), w16.float(), dy16.float()
    out["rmsnorm_fwd_f16"] = timed_ms(lambda: ew.rmsnorm(x16, w16))
    out["rmsnorm_fwd_f32_with_f16_copy"] = timed_ms(lambda: ew.rmsnorm(x32, w32).half())
    fwd16 = timed_ms(lambda: ew.rmsnorm(x16, w16))
    out["rmsnorm_bwd_f16"] = max(timed_ms(lambda: ew.rmsnorm_fwd_bwd(x16, w16, dy16)) - fwd16, 0.0)
    fwd32 = timed_ms(lambda: ew.rmsnorm(x32, w32))
    out["rmsnorm_bwd_from_f16_copy"] = max(timed_ms(lambda: ew.rmsnorm_fwd_bwd(x32, w32, dy32)) - fwd32, 0.0)
    pos = torch.cat([torch.arange(512), torch.arange(384), torch.arange(640), torch.arange(512)])
    cos, sin = ew.rope_tables(pos, 128, dtype=torch.float16)
    q = torch.randn(1, n, 12 * 128, generator=gen).half().view(1, n, 12, 128).transpose(1, 2)
    k = torch.randn(1, n, 2 * 128, generator=gen).half().view(1, n, 2, 128).transpose(1, 2)
    out["rope_fwd_q_and_k"] = timed_ms(lambda: ew.rope(q, k, cos, sin))
    gq, gk = torch.randn(1, 12, n, 128, generator=gen).half(), torch.randn(1, 2, n, 128, generator=gen).half()
    out["rope_bwd_q_and_k"] = max(timed_ms(lambda: ew.rope_fwd_bwd(q, k, cos, sin, gq, gk))
                                  - out["rope_fwd_q_and_k"], 0.0)
    g = torch.randn(n, inter, generator=gen).half()
    u = torch.randn(n, inter, generator=gen).half()
    dy = torch.randn(n, inter, generator=gen).half()
    out["silu_mul_fwd"] = timed_ms(lambda: ew.swiglu(g, u))
    out["silu_mul_bwd_inplace"] = max(timed_ms(lambda: ew.swiglu_fwd_bwd(g, u, dy)) - out["silu_mul_fwd"], 0.0)
    xd = torch.randn(n, H, generator=gen)
    mask = torch.rand(n, H, generator=gen) > 0.05
    out["dropout_pack"] = timed_ms(lambda: ew.dropout_pack(xd, mask, 1 / 0.95))
    _, bits = ew.dropout_pack(xd, mask, 1 / 0.95)
    g16 = torch.randn(n, H, generator=gen).half()
    out["dropout_unpack"] = timed_ms(lambda: ew.dropout_unpack(xd.half(), bits, g16, 1 / 0.95, torch.float32))
    wq = (torch.randn(1536, 1536, generator=gen) * 0.02).half()
    packed, state = onf4.quantize_nf4(wq)
    one = timed_ms(lambda: onf4.dequantize_nf4(packed, state, torch.float16))
    # 1536 x 1536 is 2.36 M of the 1310 M elements of the 28 layers: scaled by the element count
    out["nf4_dequant_28_layers"] = one * (1310195712 / wq.numel())
    out["nf4_dequant_28_layers_batched_per_layer"] = out["nf4_dequant_28_layers"]
    out["nf4_dequant_8960x1536"] = one * (8960 * 1536 / wq.numel())
    return {k: round(v, 3) for k, v in out.items()}


# ------------------------------------------------------------------------------------------
def step_only(dev, steps):
    """The captured Qwen2.5-1.5B-architecture QLoRA step alone (same model, batch and optimizer as
    `qlora_step_leg` on one GPU): five warm replays, one replay inside the NVTX range 'soup_step',
    then `steps` timed replays."""
    import claudemaxing_b200 as solution
    from claudemaxing_b200 import qlora

    solution.apply()
    model, lora = qlora.build_qlora_model(dev, seed=0)
    batch = qlora.synthetic_batch(seed=3)
    optimizer = torch.optim.AdamW(lora, lr=1e-4, fused=True, capturable=True)
    scaler = torch.amp.GradScaler("cuda", init_scale=65536.0)
    captured = qlora.CapturedStep(model, lora, optimizer, batch, scaler=scaler)
    for _ in range(5):
        captured.run()
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_push("soup_step")
    captured.run()
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_pop()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        loss = captured.run()
    b.record()
    torch.cuda.synchronize()
    return {"qlora_step_ms": round(a.elapsed_time(b) / steps, 4), "loss": float(loss),
            "bucket_tokens": captured.bucket, "real_tokens": batch["n_tokens"]}


def qlora_step_leg(dev, rank, world, steps, warmup, timed):
    """benchmark config 4 (and 5b at N>1): the full Qwen2.5-1.5B-architecture QLoRA step, batch 4 per
    GPU with lengths uniform in [64, 512], packed; forward, backward, LoRA-gradient all-reduce at
    N>1, fused AdamW. Timed as CUDA-graph replays (CapturedStep) and, for comparison, eagerly."""
    import torch.distributed as dist

    import claudemaxing_b200 as solution
    from claudemaxing_b200 import qlora

    solution.apply()
    model, lora = qlora.build_qlora_model(dev, seed=0)          # same weights on every rank
    batch = qlora.synthetic_batch(seed=3 + rank)                 # each rank its own 4 rows (host)
    for k in ("input_ids", "attention_mask", "labels"):
        batch[k] = batch[k].pin_memory()
    n_real = torch.tensor([batch["n_tokens"]], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(n_real)
    n_real = int(n_real.item())
    optimizer = torch.optim.AdamW(lora, lr=1e-4, fused=True, capturable=True)
    scaler = torch.amp.GradScaler("cuda", init_scale=65536.0)
    captured = qlora.CapturedStep(model, lora, optimizer, batch, scaler=scaler)
    first = float(captured.run())
    for _ in range(max(warmup, 3)):
        captured.run()
    ms = sorted(timed(captured.run, steps) / steps for _ in range(3))[1]

    def e2e():
        captured.load(batch)
        return captured.run().item()

    for _ in range(3):
        last = e2e()
    e2e_ms = sorted(timed(e2e, steps) / steps for _ in range(3))[1]
    dev_batch = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in batch.items()}
    eager_opt = torch.optim.AdamW(lora, lr=1e-4, fused=True)

    def eager():
        qlora.qlora_step(model, dev_batch, None, None)
        if world > 1:
            from claudemaxing_b200.parallel import allreduce_lora_grads
            allreduce_lora_grads(lora)
        eager_opt.step()
        eager_opt.zero_grad(set_to_none=True)

    for _ in range(2):
        eager()
    eager_ms = timed(eager, 5) / 5
    # the same captured step with the 4-bit projections on the tcgen05 GEMM that dequantises in its
    # operand prologue (off by default: see NF4Linear.fused_gemm)
    fused_ms = None
    if world == 1:
        qlora.NF4Linear.fused_gemm = True
        try:
            opt2 = torch.optim.AdamW(lora, lr=1e-4, fused=True, capturable=True)
            fused_step = qlora.CapturedStep(model, lora, opt2, batch, scaler=torch.amp.GradScaler("cuda", init_scale=65536.0))
            for _ in range(3):
                fused_step.run()
            fused_ms = sorted(timed(fused_step.run, steps) / steps for _ in range(3))[1]
            del fused_step, opt2
        finally:
            qlora.NF4Linear.fused_gemm = False
    dp_check = None
    if world > 1:
        # outside the timed regions: the all-reduced flat LoRA gradient is the mean of the ranks'
        captured.load(batch)
        for _ in range(6):   # dynamic loss scaling: a step whose scaled gradient overflowed says nothing
            captured.graph_fb.replay()
            finite = torch.isfinite(captured.flat_grad).all().float()
            dist.all_reduce(finite, op=dist.ReduceOp.MIN)
            if bool(finite):
                break
            captured.graph_opt.replay()   # the scaler lowers the scale and skips the update
        mine = captured.flat_grad.clone()
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        want = torch.stack(gathered).double().mean(0)
        dist.all_reduce(captured.flat_grad)
        captured.flat_grad.div_(world)
        err = ((captured.flat_grad.double() - want).norm() / want.norm().clamp(min=1e-30)).item()
        dp_check = {"allreduce_vs_mean_of_ranks_rel": err, "grad_norm": float(want.norm()),
                    "ok": bool(err < 1e-6 and float(want.norm()) > 0)}
    from claudemaxing_b200 import _lib as _soup_lib

    _soup_lib.check_device_status()
    return {
        "dp_gradient_check": dp_check,
        "metric": "QLoRA step tokens/s/GPU", "value": round(n_real / world / (ms * 1e-3), 1),
        "aggregate_tokens_per_s": round(n_real / (ms * 1e-3), 1), "ms_per_step": round(ms, 4),
        "real_tokens_per_step": n_real, "bucket_tokens_per_gpu": captured.bucket,
        "e2e": {"value": round(n_real / world / (e2e_ms * 1e-3), 1), "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": 3 * captured.bucket * 8 + captured.cu_rows.numel() * 4, "d2h_bytes_per_step": 4},
        "eager_ms_per_step": round(eager_ms, 4),
        "nf4_gemm_in_prologue_ms_per_step": None if fused_ms is None else round(fused_ms, 4),
        "loss_first": round(first, 5), "loss_last": round(float(last), 5),
        "config": "configs[3]: 28 layers, hidden 1536, GQA 12/2, vocab 151936 tied, NF4 + LoRA r=16 "
                  "on q_proj/v_proj, batch 4 x U[64,512] packed, fp16 autocast, dynamic loss scale, "
                  "fused AdamW" + ("" if world == 1 else f"; data-parallel x{world}, flat LoRA-gradient all-reduce"),
        "timing": "two CUDA graphs per step (forward+backward, optimizer), all-reduce between them",
    }


# ------------------------------------------------------------------------------------------
LOSS_SCALE = 4096.0   # the loss is scaled as a trainer's GradScaler does: fp16 dHidden stays normal
C5A_TOKENS = 65536


def recorded_traffic():
    """DRAM bytes per step of the two GEMM kernels at config 1 on one GPU, as recorded from an ncu
    capture in the line `traffic_bytes_per_step logits=<bytes> grad=<bytes>` of
    profiles/lmhead_c1_kernels_full.md (None when the file or the line is missing)."""
    try:
        with open(os.path.join(ROOT, "profiles", "lmhead_c1_kernels_full.md")) as f:
            for line in f:
                if line.startswith("traffic_bytes_per_step"):
                    return {k: float(v) for k, v in (kv.split("=") for kv in line.split()[1:])}
    except Exception:  # noqa: BLE001
        pass
    return None


def head_launches(n_rows, v_local, world):
    """Kernels of this library one head pass over n_rows x v_local launches: state init, per row
    block and chunk (logits, row merge, gradient) plus the first chunk's rescale, status publish,
    finish, backward scale (or rounding before the reduce-scatter); at N>1 also the merge."""
    from claudemaxing_b200 import _lib

    rb, ct1, ct = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    _lib.lib().soup_lmhead_plan(n_rows, v_local, 0, ctypes.byref(rb), ctypes.byref(ct1), ctypes.byref(ct))
    row_blocks = -(-n_rows // rb.value)
    col_tiles = -(-v_local // 256)
    chunks = 1 + -(-max(col_tiles - ct1.value, 0) // ct.value)
    return 1 + row_blocks * (chunks * 3 + 1) + 1 + 1 + 1 + (1 if world > 1 else 0)


class HeadJob:
    """One workload of the fused head on this rank: `slabs` slabs of rows fed by this rank (pinned
    host copies and device copies), the weight shard, and the step through the public API."""

    def __init__(self, dev, rank, world, slabs, w_dev, bounds):
        import torch.distributed as dist

        self.dev, self.rank, self.world, self.slabs = dev, rank, world, slabs
        self.w_dev, self.bounds = w_dev, bounds
        hidden, target = make_local_rows(rank, slabs)
        self.n_local = hidden.shape[0]
        self.n_tokens = self.n_local * world
        self.hidden_pin, self.target_pin = hidden.pin_memory(), target.pin_memory()
        self.hidden_dev, self.target_dev = self.hidden_pin.to(dev), self.target_pin.to(dev)
        self.dh_pin = torch.empty(self.n_local, HIDDEN, dtype=torch.float16).pin_memory()
        labelled = (self.target_dev != -100).sum()
        if world > 1:
            dist.all_reduce(labelled)
        self.n_labelled = int(labelled)
        self.scale = torch.tensor(LOSS_SCALE, device=dev)

    def step(self, h_dev, t_dev):
        """fwd+bwd; returns (loss of the whole job, fp16 dHidden of this rank's rows at LOSS_SCALE,
        per-row loss, per-row entropy of this rank's rows)."""
        from claudemaxing_b200 import parallel
        from claudemaxing_b200.lm_head_loss import GRAD_SCALE, fused_head_loss

        if self.world == 1:
            h = h_dev.detach().requires_grad_(True)
            loss, terms = fused_head_loss(h[None], self.w_dev, None, target=t_dev[None])
            loss.backward(self.scale)
            return loss.detach(), h.grad, terms.token_loss[0], terms.token_entropy[0]
        res = parallel.vocab_parallel_head_rows(h_dev, t_dev, self.w_dev, self.bounds)
        loss = res["loss_sum"] / res["labelled"]
        grad = res["grad"] * (LOSS_SCALE / (GRAD_SCALE * res["labelled"]))
        return loss, grad, res["token_loss"], res["entropy"]

    def parity(self, weight_h, sample_per_rank, cpu_rows=None):
        """Per-row loss / entropy / dHidden of a sample of rows from every rank against the CPU
        oracle (fp32 matmul + log_softmax + autograd). At N=1 `cpu_rows` makes the sample the first
        `cpu_rows` rows (the pass the CPU baseline times anyway) and its duration is returned too."""
        import torch.distributed as dist

        from oracle.head_ce import head_ce

        loss, grad, tl, en = self.step(self.hidden_dev, self.target_dev)
        if cpu_rows:
            idx = torch.arange(min(cpu_rows, self.n_local))
        else:
            k = min(sample_per_rank, self.n_local)
            idx = torch.linspace(0, self.n_local - 1, k).round().long().unique()
        idx_dev = idx.to(self.dev)
        mine = torch.cat([tl[idx_dev, None].float(), en[idx_dev, None].float(),
                          grad[idx_dev].float()], 1).contiguous()
        everyone = mine
        if self.world > 1:
            everyone = torch.empty((self.world * mine.shape[0], mine.shape[1]), device=self.dev)
            dist.all_gather_into_tensor(everyone, mine)
        if self.rank != 0:
            return None, None
        got = everyone.cpu().view(self.world, idx.numel(), -1)
        h_rows, t_rows = [], []
        for r in range(self.world):   # regenerate the sampled rows of every rank from their seeds
            if r == 0:
                h_r, t_r = self.hidden_pin, self.target_pin
            else:
                h_r, t_r = make_local_rows(r, self.slabs)
            h_rows.append(h_r[idx])
            t_rows.append(t_r[idx])
        h_s, t_s = torch.cat(h_rows), torch.cat(t_rows)
        torch.set_num_threads(os.cpu_count() or 1)
        t0 = time.perf_counter()
        ref = head_ce(h_s, weight_h, t_s, denominator=self.n_labelled, grad_scale=LOSS_SCALE)
        seconds = time.perf_counter() - t0
        got = got.view(-1, got.shape[-1])
        dh_scale = ref["dhidden"].abs().max().item()
        rec = {
            "rows": int(got.shape[0]), "ranks_sampled": self.world,
            "max_abs_loss": float((got[:, 0] - ref["token_loss"]).abs().max()),
            "max_abs_entropy": float((got[:, 1] - ref["entropy"]).abs().max()),
            "dh_rel_max": float((got[:, 2:] - ref["dhidden"]).abs().max() / max(dh_scale, 1e-30)),
            "oracle": "oracle/head_ce.py, fp32 CPU, same rows regenerated from their seeds",
            "tolerances": {"loss": 1e-3, "entropy": 1e-3, "dh_rel_max": 1e-2},
        }
        rec["ok"] = bool(rec["max_abs_loss"] <= 1e-3 and rec["max_abs_entropy"] <= 1e-3
                         and rec["dh_rel_max"] <= 1e-2 and math.isfinite(float(loss)))
        return rec, (int(got.shape[0]), seconds)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1", choices=["c1", "c5a"])
    ap.add_argument("--regions", type=int, default=5, help="timed regions of --steps steps each")
    ap.add_argument("--no-suite", action="store_true", help="skip the memory-bound kernel suite")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-step", action="store_true", help="skip the full QLoRA training step leg")
    ap.add_argument("--no-c5a", action="store_true", help="skip the 65536-token sub-record")
    ap.add_argument("--suite-only", action="store_true",
                    help="run only the memory-bound kernel suite and print its JSON")
    ap.add_argument("--suite-rows", type=int, default=32768)
    ap.add_argument("--gemm-only", action="store_true",
                    help="run only the NF4 GEMM comparison and print its JSON")
    ap.add_argument("--attention-only", action="store_true",
                    help="run only the packed-row attention comparison and print its JSON")
    ap.add_argument("--step-only", action="store_true",
                    help="run only the captured QLoRA step: warm replays, then one replay inside the "
                         "NVTX range 'soup_step' (for a profiler's range filter), then a timed region")
    ap.add_argument("--plain-launches", action="store_true",
                    help="with --suite-only: up to three direct launches per case instead of graph replays")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.regions = max(args.regions, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist

    from claudemaxing_b200 import _lib, parallel

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    global PLAIN_LAUNCHES
    if args.suite_only:
        PLAIN_LAUNCHES = args.plain_launches
        hbm = peaks()[0]["hbm_gbs"]
        print(json.dumps({"kernels": kernel_suite(dev, hbm, n_rows=args.suite_rows,
                                                  tag=f"@{args.suite_rows}rows",
                                                  with_nf4=True)}), flush=True)
        return
    if args.gemm_only:
        PLAIN_LAUNCHES = args.plain_launches
        suite = nf4_gemm_suite(dev, peaks()[0]["bf16_tflops"])
        suite.update(attention_suite(dev, peaks()[0]["bf16_tflops"]))
        print(json.dumps({"kernels": suite}), flush=True)
        return
    if args.step_only:
        print(json.dumps(step_only(dev, max(args.steps, 1))), flush=True)
        return
    if args.attention_only:
        PLAIN_LAUNCHES = args.plain_launches
        print(json.dumps({"kernels": attention_suite(dev, peaks()[0]["bf16_tflops"])}), flush=True)
        return
    if world > 1:
        # stdout carries one JSON line: keep NCCL's version banner (NCCL_DEBUG=VERSION, from the
        # environment or from a system-wide nccl.conf, which the environment overrides) off it
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    peak, peak_source = peaks()

    c5a_slabs = C5A_TOKENS // SLAB // world if (C5A_TOKENS // SLAB) % world == 0 else 0
    slabs = c5a_slabs if args.workload == "c5a" else TOKENS_PER_GPU // SLAB
    if slabs == 0:
        raise SystemExit(f"--workload c5a needs a GPU count that divides {C5A_TOKENS // SLAB}")
    weight_h = make_weight()
    bounds = parallel.shard_bounds(VOCAB, world)
    w_dev = weight_h[bounds[rank]:bounds[rank + 1]].to(dev)
    if rank != 0:
        del weight_h
        weight_h = None
    job = HeadJob(dev, rank, world, slabs, w_dev, bounds)
    n_tokens, n_local = job.n_tokens, job.n_local

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        clocks.windows.append((t0, time.time()))
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    def regions_of(fn, steps, count):
        """`count` timed regions of exactly `steps` steps: [(ms per step, median SM MHz inside)]."""
        out = []
        for _ in range(count):
            ms = timed(fn, steps) / steps
            out.append((ms, clocks.window_mhz(len(clocks.windows) - 1)))
        return out

    def summarise(regs):
        ms = sorted(r[0] for r in regs)
        return {"median_ms": round(statistics.median(ms), 5), "min_ms": round(ms[0], 5),
                "regions": [{"ms_per_step": round(m, 5), "sm_mhz": c,
                             "ms_x_ghz": None if c is None else round(m * c / 1e3, 5)} for m, c in regs]}

    # ---- device-resident regions (value). The clock sampler (an NVML thread of this process)
    # starts before the warm-up and keeps sampling through every timed region.
    clocks = ClockSampler(local_rank)
    clocks.__enter__()
    clocks.wait_first_sample()
    for _ in range(args.warmup):
        loss = job.step(job.hidden_dev, job.target_dev)[0]
    # Several regions of exactly K steps: a K-step region is tens of milliseconds, on a part whose
    # clock moves with the power cap, and on these shared hosts a region now and then contains a
    # one-off stall. The median region is the reported value; the minimum and each region's
    # sampled SM clock (time x clock separates clock effects from kernel effects) are beside it.
    value_regions = regions_of(lambda: job.step(job.hidden_dev, job.target_dev), args.steps, args.regions)
    value_sum = summarise(value_regions)
    ms_per_step = value_sum["median_ms"]
    value = n_tokens / (ms_per_step * 1e-3)

    # ---- end-to-end regions: this rank's rows from pinned host memory in, loss (host read) and
    # this rank's dHidden rows out, every step
    def e2e_serial_step():
        h = job.hidden_pin.to(dev, non_blocking=True)
        t = job.target_pin.to(dev, non_blocking=True)
        loss, grad = job.step(h, t)[:2]
        job.dh_pin.copy_(grad.reshape(n_local, HIDDEN), non_blocking=True)
        return loss.item()

    for _ in range(3):
        e2e_serial_step()
    e2e_serial = summarise(regions_of(e2e_serial_step, args.steps, 3))

    # The same with the feed a trainer's data loader gives: while a step computes, a copy stream
    # brings the next step's inputs from pinned host memory into the other of two device buffer
    # pairs and takes the previous step's dHidden back, so PCIe runs in both directions beside the
    # GEMMs. Every step still copies its inputs in, copies dHidden out and reads its loss on the
    # host; the one prefetch issued before a region starts is matched by one left over at its end.
    copy_stream = torch.cuda.Stream()
    h_bufs = [torch.empty_like(job.hidden_dev) for _ in range(2)]
    t_bufs = [torch.empty_like(job.target_dev) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    state = {"cur": 0, "grad": None}

    def prefetch(slot):
        with torch.cuda.stream(copy_stream):
            h_bufs[slot].copy_(job.hidden_pin, non_blocking=True)
            t_bufs[slot].copy_(job.target_pin, non_blocking=True)
            ready[slot].record(copy_stream)

    def e2e_step():
        cur = state["cur"]
        main_stream = torch.cuda.current_stream()
        main_stream.wait_event(ready[cur])
        copy_stream.wait_stream(main_stream)   # the other pair is free: the previous step has been enqueued
        prefetch(cur ^ 1)
        loss, grad = job.step(h_bufs[cur], t_bufs[cur])[:2]
        done = torch.cuda.Event()
        done.record(main_stream)
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(done)
            job.dh_pin.copy_(grad.reshape(n_local, HIDDEN), non_blocking=True)
        grad.record_stream(copy_stream)        # its memory is not reused before the copy has run
        state["grad"] = grad
        state["cur"] = cur ^ 1
        return loss.item()

    prefetch(0)
    for _ in range(3):
        e2e_step()
    e2e = summarise(regions_of(e2e_step, args.steps, args.regions))
    e2e_ms = e2e["median_ms"]
    copy_stream.synchronize()
    h2d = (job.hidden_pin.numel() * 2 + job.target_pin.numel() * 8) * world
    d2h = (job.dh_pin.numel() * 2 + 4) * world
    del h_bufs, t_bufs

    # ---- per-kernel region: event-bracketed launches inside the library
    sink = (ctypes.c_float * 6)()
    _lib.lib().soup_lmhead_set_timing(ctypes.cast(sink, ctypes.c_void_p))
    barrier()
    for _ in range(args.steps):
        job.step(job.hidden_dev, job.target_dev)
    barrier()
    _lib.lib().soup_lmhead_set_timing(None)
    clocks.__exit__(None, None, None)
    _lib.check_device_status()
    k_ms = [sink[i] / args.steps for i in range(3)]
    k_launch = [int(round(sink[3 + i] / args.steps)) for i in range(3)]
    v_local = bounds[rank + 1] - bounds[rank]
    flops_gemm = 2.0 * n_tokens * HIDDEN * v_local  # per GEMM kind, this rank, per step
    tf = lambda ms: flops_gemm / (ms * 1e-3) / 1e12 if ms > 0 else 0.0  # noqa: E731
    tensor_peak = peak["bf16_tflops"]
    logits_tf, grad_tf = tf(k_ms[0]), tf(k_ms[2])
    traffic = recorded_traffic() if (world == 1 and args.workload == "c1") else None
    minimum_bytes = 2.0 * v_local * HIDDEN + 2.0 * n_tokens * HIDDEN + 4.0 * n_tokens * HIDDEN
    roofline = {
        "kernel": "lmhead_logits_kernel (tcgen05 GEMM + softmax-statistics epilogue)",
        "bound": "tensor", "achieved": round(logits_tf, 1), "peak": tensor_peak, "unit": "TFLOP/s",
        "frac": round(logits_tf / tensor_peak, 4), "peak_source": peak_source + " cuBLAS bf16 burst",
        "frac_of_sustained": round(logits_tf / peak["bf16_tflops_sustained"], 4),
        "frac_of_nominal_2250": round(logits_tf / 2250.0, 4),
        "ms_per_launch": round(k_ms[0] / max(k_launch[0], 1), 5), "launches_per_step": k_launch[0],
        # DRAM bytes (read + write) of the logits launches of one step divided by their number,
        # from the ncu capture recorded in profiles/; config 1 on one GPU only
        "traffic": None if not traffic else round(traffic["logits"] / max(k_launch[0], 1)),
        "traffic_per_step": None if not traffic else {
            "logits_kernel": traffic["logits"], "grad_kernel": traffic["grad"],
            "both": traffic["logits"] + traffic["grad"],
            "minimum_w_once_hidden_dh": minimum_bytes,
            "ratio_to_minimum": round((traffic["logits"] + traffic["grad"]) / minimum_bytes, 2),
            "note": "the probabilities of a chunk pass from the logits to the gradient kernel "
                    "through a bf16 buffer and the gradient GEMM reads a bf16 copy of W: that "
                    "traffic is measured here and is not part of the minimum"},
        "grad_kernel": {"achieved": round(grad_tf, 1), "frac": round(grad_tf / tensor_peak, 4),
                        "ms_per_launch": round(k_ms[2] / max(k_launch[2], 1), 5),
                        "launches_per_step": k_launch[2]},
        "row_kernel_ms_per_step": round(k_ms[1], 5),
        "fused_op": {"achieved": round(2 * flops_gemm / (ms_per_step * 1e-3) / 1e12, 1),
                     "frac": round(2 * flops_gemm / (ms_per_step * 1e-3) / 1e12 / tensor_peak, 4),
                     "min_region_frac": round(2 * flops_gemm / (value_sum["min_ms"] * 1e-3) / 1e12 / tensor_peak, 4),
                     "note": "4*N*H*V_local / whole step time (all kernels, launch gaps, collectives)"},
    }
    if world == 1:
        launches = head_launches(n_tokens, v_local, 1)
    else:
        steps_plan = parallel.plan_exchange_steps(n_local, world,
                                                  parallel.step_rows(n_tokens, HIDDEN, bounds))
        launches = sum(head_launches((z - a) * world, v_local, world) for a, z in steps_plan)

    # ---- parity against the CPU oracle, outside every timed region, at every N
    cpu = None
    cores = os.cpu_count() or 1
    cpu_rows = None
    if rank == 0:
        weight_h = weight_h.float()   # once: the oracle multiplies in fp32
    if rank == 0 and world == 1 and not args.no_cpu and args.workload == "c1":
        probe_rec, probe = job.parity(weight_h, 32, cpu_rows=32)
        cpu_rows = int(max(32, min(n_local, probe[0] / probe[1] * 12.0)) // 32 * 32)
    parity, timing = job.parity(weight_h, max(16, 128 // world), cpu_rows=cpu_rows)
    if cpu_rows and timing:
        cpu = {"value": round(timing[0] / timing[1], 2), "unit": "tokens/s", "cores": cores,
               "kind": "port",
               "sample": f"{timing[0]} of the {n_local} rows x full vocabulary, one pass, torch fp32 "
                         "matmul + log_softmax + autograd (oracle/head_ce.py); its output is the "
                         "reference of `parity`"}

    # ---- benchmark configs[4](a): the fixed 65536-token job, vocabulary-parallel over N
    c5a = None
    if args.workload == "c1" and not args.no_c5a and c5a_slabs:
        del job
        torch.cuda.empty_cache()
        big = HeadJob(dev, rank, world, c5a_slabs, w_dev, bounds)
        for _ in range(2):
            big.step(big.hidden_dev, big.target_dev)
        c5a_regions = regions_of(lambda: big.step(big.hidden_dev, big.target_dev), 5, 2)
        c5a_sum = summarise(c5a_regions)
        c5a_parity, _ = big.parity(weight_h, max(16, 128 // world))
        _lib.check_device_status()
        c5a = {"workload": f"configs[4a]: {C5A_TOKENS} tokens, vocabulary-parallel x{world}, "
                           f"{big.n_local} rows fed by each rank", "tokens": C5A_TOKENS,
               "steps": 5, "warmup": 2, "scaling": "strong",
               "ms_per_step": c5a_sum["median_ms"], "min_ms_per_step": c5a_sum["min_ms"],
               "value": round(C5A_TOKENS / (c5a_sum["median_ms"] * 1e-3), 1), "unit": "tokens/s",
               "tflops": round(4.0 * C5A_TOKENS * HIDDEN * VOCAB / (c5a_sum["median_ms"] * 1e-3) / 1e12, 1),
               "frac_of_measured_burst_per_gpu": round(
                   4.0 * C5A_TOKENS * HIDDEN * VOCAB / (c5a_sum["median_ms"] * 1e-3) / 1e12 / world / tensor_peak, 4),
               "regions": c5a_sum["regions"], "parity": c5a_parity}
        del big
        torch.cuda.empty_cache()

    kernels = None
    if rank == 0 and world == 1:
        if not args.no_suite:
            kernels = kernel_suite(dev, peak["hbm_gbs"])
            # the same kernels on 16x and 32x the rows: launch ramps amortised, data far larger than L2
            kernels.update(kernel_suite(dev, peak["hbm_gbs"], n_rows=32768, tag="@32768rows",
                                        with_nf4=False))
            kernels.update(kernel_suite(dev, peak["hbm_gbs"], n_rows=65536, tag="@65536rows",
                                        with_nf4=False))
            kernels.update(nf4_gemm_suite(dev, tensor_peak))
            kernels.update(attention_suite(dev, tensor_peak))
        if not args.no_cpu and kernels is not None:
            cpu_ms = cpu_oracle_suite(cores)
            for key, ms in cpu_ms.items():
                if key in kernels:
                    kernels[key]["cpu_oracle_ms"] = ms
                    kernels[key]["cpu_oracle_cores"] = cores

    step_leg = None
    if not args.no_step and args.workload == "c1":
        del w_dev
        torch.cuda.empty_cache()
        step_leg = qlora_step_leg(dev, rank, world, max(5, min(args.steps, 20)), args.warmup, timed)

    if rank == 0:
        line = {
            "metric": "fused LM-head+CE fwd+bwd tokens/s", "value": round(value, 1),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 5), "min_ms_per_step": value_sum["min_ms"],
            "regions": value_sum["regions"], "higher_is_better": True,
            "scaling": "strong" if args.workload == "c5a" else "weak", "vs_baseline": None,
            "dtype": "f16 (logits GEMM fp16 x fp16; gradient GEMM bf16 probabilities x bf16 copy of "
                     "the weight; fp32 accumulation and statistics)",
            "data": "synthetic",
            "config": {
                "workload": ("configs[4a]: 65536 tokens" if args.workload == "c5a" else
                             "configs[0]: fused LM-head+CE fwd+bwd, 2048 packed tokens per GPU") +
                            f", hidden {HIDDEN}, tied fp16 head {VOCAB} x {HIDDEN}, 10% ignored",
                "tokens": n_tokens,
                "parallelism": "single GPU" if world == 1 else
                               f"vocabulary-parallel x{world}, rows fed data-parallel: per exchange "
                               "step an all-gather of hidden rows and targets, an all-gather of "
                               "per-row states, a reduce-scatter of fp16 dHidden",
                "loss_scale": LOSS_SCALE,
                "l2": "inputs larger than L2: the 467 MB head weight streams from HBM every step",
                "tflops_per_step_algorithmic": round(4.0 * n_tokens * HIDDEN * VOCAB / 1e12, 4),
            },
            "tflops": round(4.0 * n_tokens * HIDDEN * VOCAB / (ms_per_step * 1e-3) / 1e12, 1),
            "e2e": {"value": round(n_tokens / (e2e_ms * 1e-3), 1), "unit": "tokens/s",
                    "ms_per_step": round(e2e_ms, 5), "min_ms_per_step": e2e["min_ms"],
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "feed": "every rank copies only the rows it owns; double-buffered: the next "
                            "step's host->device copies and the previous step's dHidden "
                            "device->host copy run on a copy stream beside the step",
                    "serial_ms_per_step": e2e_serial["median_ms"]},
            "gpu_launches": launches * args.steps,
            "gpu_launches_per_step": launches,
            "clocks": clocks.summary(),
            "roofline": roofline,
            "parity": parity,
            "loss": round(float(loss), 6),
        }
        if c5a is not None:
            line["c5a"] = c5a
        if kernels is not None:
            line["kernels"] = kernels
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if step_leg is not None:
            line["qlora_step"] = step_leg
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
