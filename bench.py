#!/usr/bin/env python
"""Benchmark of the WKV7 time-mix hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (N = 1 and every N): recurrent decode at B=256 sequences, H=32, D=64,
bf16 tokens, fp32 state pool read and written in place.  One benchmark *step* is
one pass over a batch of synthetic input: 256 consecutive decode steps of the 256
sequences (65 536 tokens, 256 kernel launches per rank).  With N GPUs the 256
sequences are split into contiguous blocks of 256/N per rank, each rank owning its
slice of the state pool (strong scaling, no collective on the data path); `value`
is the job's tokens/s using the slowest rank's time.  For N > 1 `extras` adds the
timed all-gather of one step's outputs, the weak-scaling figure (256 sequences per
rank) and the chunked prefill with its 8 sequences split over the ranks.

The line printed by rank 0 carries, besides the contract keys, `roofline`
(algorithmic bytes per launch / measured launch time against the measured HBM
peak), `cpu_baseline` (the CPU oracle timed on the host cores) and `e2e` (the same
metric with host buffers: pinned-host -> device copies of every decode step's six
token tensors and a device -> host read of its output inside the timed region).

`--impl reference` times the CPU port of the reference's recurrence (the oracle)
on a bounded sample and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

B, H, D = 256, 32, 64
DECODE_STEPS_PER_STEP = 256          # "run 256 consecutive steps"
TOKEN_RING = 8                       # distinct pre-generated decode steps of token data
METRIC = "WKV7 recurrent decode tokens/s (B=256,H=32,D=64, fp32 state in place)"
# algorithmic bytes of one decode launch: per (sequence, head) 2*D*D*4 (state read + write)
# + 7*D*2 (r,w,k,v,a,b in, y out)
BYTES_PER_UNIT = 2 * D * D * 4 + 7 * D * 2
BYTES_PER_LAUNCH = B * H * BYTES_PER_UNIT
FALLBACK_HBM_GBS = 6650.0


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the bench runs."""

    def __init__(self, index: int):
        self.samples = []
        self.timed = False
        self._stop = threading.Event()
        self._thread = None
        self.sm_max = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                self.samples.append((self.timed, mhz, int(reasons)))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def summary(self):
        if self._nv is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["nvml unavailable"]}
        timed = [s for s in self.samples if s[0]] or self.samples
        nv = self._nv
        names = {
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        seen = sorted(n for n, bit in names.items() if any(s[2] & bit for s in timed))
        return {"sm_mhz": statistics.median(s[1] for s in timed), "sm_max_mhz": self.sm_max,
                "reasons": seen, "samples": len(timed)}


class CpuPort:
    """The CPU oracle (C port of the reference recurrence, OpenMP over (sequence, head))."""

    def __init__(self):
        from flashrwkv_b200 import synthetic
        from oracle import wkv7_oracle

        wkv7_oracle.build()
        # launchers such as torchrun export OMP_NUM_THREADS=1: the CPU arm is meant to use every core it may run on
        wkv7_oracle.set_num_threads(len(os.sched_getaffinity(0)))
        self.oracle = wkv7_oracle
        self.cu, self.idx = synthetic.equal_length_metadata(B, 1)
        self.pool = synthetic.state_pool(B, H, D, seed=1).numpy()
        self.toks = [t.float().numpy() for t in synthetic.wkv7_inputs(B, H, D, seed=2)]
        self.toks16 = synthetic.wkv7_inputs(B, H, D, seed=2)

    def decode_steps(self, n: int) -> float:
        """Run n decode steps of the batch; return the seconds they took."""
        t0 = time.perf_counter()
        for _ in range(n):
            self.oracle.forward(*self.toks, state_pool=self.pool, cu_seqlens=self.cu, state_indices=self.idx,
                                double=False, inplace=True)
        return time.perf_counter() - t0

    def pytorch_port_tokens_per_s(self, reps: int = 2) -> float:
        """The oracle in the reference's own form: pure PyTorch, Python loop over sequences and tokens."""
        import torch

        tp = torch.from_numpy(self.pool)
        t0 = time.perf_counter()
        for _ in range(reps):
            _, tp = self.oracle.forward_torch(*self.toks16, state_pool=tp, cu_seqlens=self.cu,
                                              state_indices=self.idx)
        return B * reps / (time.perf_counter() - t0)

    def describe(self, value: float, sample: str) -> dict:
        import torch

        return {"value": value, "unit": "tokens/s", "cores": self.oracle.num_threads(), "kind": "port",
                "sample": sample, "pytorch_port_tokens_per_s": self.pytorch_port_tokens_per_s(),
                "pytorch_port_threads": torch.get_num_threads(), "host_cpus": os.cpu_count()}


def _cpu_baseline(sample_decode_steps: int) -> dict:
    port = CpuPort()
    port.decode_steps(2)
    dt = port.decode_steps(sample_decode_steps)
    return port.describe(B * sample_decode_steps / dt,
                         f"{sample_decode_steps} decode steps of the same B={B},H={H},D={D} batch; fp32 C port of "
                         f"the reference recurrence, OpenMP over (sequence, head)")


def run_reference(args):
    """The CPU arm: each step is a bounded sample (16 decode steps) of the workload."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    sample = 16
    port = CpuPort()
    for _ in range(args.warmup):
        port.decode_steps(sample)
    dt = sum(port.decode_steps(sample) for _ in range(args.steps))
    value = B * sample * args.steps / dt
    base = port.describe(value, f"{args.steps} steps x {sample} decode steps of the B={B},H={H},D={D} batch; fp32 C "
                                f"port of the reference recurrence, OpenMP over (sequence, head)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"recurrent decode B={B} H={H} D={D}, fp32 state, CPU port of the reference "
                               f"recurrence; each step = {sample} decode steps (bounded sample)"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _time_cuda(fn, warmup=2, iters=5):
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def _extras_glue(dev, hbm):
    """Training-side TMix glue kernels, each timed alone; hbm = the peak in bytes/s the fractions are quoted against."""
    import torch

    # ---- training-side TMix glue on the training configuration's activations: B=8, T=4096, C=4096 (268 MB per tensor,
    # larger than L2).  Algorithmic bytes per element = 2 x the tensors read or written.
    from flashrwkv_b200 import _ext

    ext = _ext.extension()
    Bt, Tt, Ct = 8, 4096, 4096
    gen = torch.Generator(device=dev).manual_seed(9)
    acts = [torch.randn(Bt, Tt, Ct, device=dev, generator=gen).to(torch.bfloat16) for _ in range(7)]
    x, r, k, v, gg, go, aa = acts
    vecs = [torch.rand(Ct, device=dev, generator=gen).to(torch.bfloat16) for _ in range(6)]
    inv = ext.pretrain_tmix_kk_pre_forward(x, vecs[0], r, vecs[1], 64)[3]
    stats = ext.pretrain_tmix_lnx_rkvres_xg_forward(x, r, k, v, vecs[0], vecs[1], vecs[2], gg, 64)[1:]
    cases = {
        "a_gate_forward": (4, lambda: ext.pretrain_tmix_a_gate_forward(vecs[0], x)),
        "a_gate_backward": (6, lambda: ext.pretrain_tmix_a_gate_backward(go, vecs[0], x)),
        "vres_gate_backward": (14, lambda: ext.pretrain_tmix_vres_gate_backward(go, x, r, vecs[0], k)),
        "mix6_forward": (14, lambda: ext.pretrain_tmix_mix6_forward(x, *vecs)),
        "mix6_backward": (16, lambda: ext.pretrain_tmix_mix6_backward(x, r, k, v, gg, go, aa, *vecs)),
        "kk_pre_forward": (10, lambda: ext.pretrain_tmix_kk_pre_forward(x, vecs[0], r, vecs[1], 64)),
        "kk_pre_backward": (14, lambda: ext.pretrain_tmix_kk_pre_backward(k, v, gg, x, vecs[0], r, vecs[1], inv, 64)),
        "lnx_rkvres_xg_forward": (12, lambda: ext.pretrain_tmix_lnx_rkvres_xg_forward(x, r, k, v, vecs[0], vecs[1],
                                                                                      vecs[2], gg, 64)),
        "lnx_rkvres_xg_backward": (22, lambda: ext.pretrain_tmix_lnx_rkvres_xg_backward(
            go, x, r, k, v, vecs[0], vecs[1], vecs[2], gg, stats[0], stats[1], 64)),
    }
    glue = {"workload": f"B={Bt} T={Tt} C={Ct} bf16, head size 64; every tensor larger than L2"}
    for name, (bytes_per_elem, fn) in cases.items():
        sec = _time_cuda(fn, warmup=2, iters=5)
        alg = Bt * Tt * Ct * bytes_per_elem
        glue[name] = {"us": sec * 1e6, "algorithmic_gbs": alg / sec / 1e9, "hbm_frac": alg / sec / hbm}
    return glue


def _extras(dev):
    """Secondary workloads of the same path, timed briefly on this GPU: chunked prefill (B8 T4096 H32), training
    forward+backward (B8 T4096 H64) and the TMix layer chain (C=2048, M in {1,4,7,512}).  Roofline fractions use
    the algorithmic bytes / FLOPs stated beside each workload and the measured peaks."""
    import torch

    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata, wkv7_chunk_forward

    out = {}
    peaks = {}
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    hbm = float(peaks.get("hbm_gbs", FALLBACK_HBM_GBS)) * 1e9
    bf16 = float(peaks.get("bf16_tflops", 1590.0)) * 1e12
    # ---- decode on an fp16 state pool (the reference's production decode contract): same batch as the headline
    cu1, idx1 = (t.to(dev) for t in synthetic.equal_length_metadata(B, 1))
    pool16 = synthetic.state_pool(B, H, D, seed=21, device=dev).half()
    elapsed = torch.zeros(B, dtype=torch.int32, device=dev)
    ring16 = [[t.to(dev) for t in synthetic.wkv7_inputs(B, H, D, seed=700 + i)] for i in range(TOKEN_RING)]
    n_steps = 128
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):  # the steps as one CUDA graph, as for the headline
        ticket16 = F.prepare_recurrent_metadata(cu1, idx1, total_tokens=B, state_pool_size=B, max_seqlen=1)

        def decode16_steps():
            for i in range(n_steps):
                F.infer_recurrent_fp16_forward_varlen(*ring16[i % TOKEN_RING], state_pool=pool16,
                                                      elapsed_state_pool=elapsed, cu_seqlens=cu1, state_indices=idx1,
                                                      max_seqlen=1, validated_metadata=ticket16)
                F.infer_recurrent_fp16_advance_i32(elapsed, 1)

        F.infer_recurrent_fp16_forward_varlen(*ring16[0], state_pool=pool16, elapsed_state_pool=elapsed,
                                              cu_seqlens=cu1, state_indices=idx1, max_seqlen=1,
                                              validated_metadata=ticket16)
        torch.cuda.synchronize(dev)
        graph16 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph16, stream=side):
            decode16_steps()
    torch.cuda.current_stream(dev).wait_stream(side)
    decode16 = graph16.replay

    sec = _time_cuda(decode16) / n_steps
    bytes16 = B * H * (2 * D * D * 2 + 7 * D * 2)
    out["decode_fp16_state"] = {
        "workload": f"recurrent decode B={B} H={H} D={D}, bf16 tokens, fp16 state pool with dither, counters advanced "
                    f"every step", "tokens_per_s": B / sec, "us_per_step": sec * 1e6,
        "algorithmic_bytes_per_launch": bytes16, "hbm_frac_algorithmic": bytes16 / sec / hbm,
        "gpu_launches_per_step": 2, "launch": f"one CUDA graph of {n_steps} steps"}
    del graph16, decode16, pool16, ring16
    # ---- chunked prefill
    Bc, T, Hc = 8, 4096, 32
    toks = [t.to(dev) for t in synthetic.wkv7_inputs(Bc * T, Hc, D, seed=11)]
    cu, _ = synthetic.equal_length_metadata(Bc, T, device=dev)
    meta = make_chunk_metadata(cu, 64)
    pool = synthetic.state_pool(Bc, Hc, D, seed=12, device=dev)
    sec = _time_cuda(lambda: wkv7_chunk_forward(*toks, state=pool, chunk_metadata=meta))
    n_tok = Bc * T
    alg_bytes = 7 * n_tok * Hc * D * 2 + 2 * Bc * Hc * D * D * 4
    flops = n_tok * Hc * 98304
    out["chunked_prefill"] = {
        "workload": f"B={Bc} T={T} H={Hc} D={D} chunk 64, bf16 tokens, fp32 state", "tokens_per_s": n_tok / sec,
        "ms": sec * 1e3, "hbm_frac_algorithmic": alg_bytes / sec / hbm, "tensor_frac_of_bf16_peak": flops / sec / bf16,
        "tensor_frac_of_tf32_peak": flops / sec / (bf16 / 2), "gpu_launches_per_call": 1,
        "kernel": "wkv7_chunk_fused_kernel"}
    del toks, pool
    # ---- training forward + backward
    Ht = 64
    toks = [t.to(dev).requires_grad_() for t in synthetic.wkv7_inputs(Bc * T, Ht, D, seed=13)]
    S0 = synthetic.state_pool(Bc, Ht, D, seed=14, device=dev).requires_grad_()
    dy = torch.randn(Bc * T, Ht, D, device=dev).to(torch.bfloat16)

    def train_step():
        res = F.statetune_recurrent_fp32io16(S0, *meta, *toks)
        res[0].backward(dy)
        for t in (*toks, S0):
            t.grad = None

    sec = _time_cuda(train_step, warmup=1, iters=2)
    out["training_fwd_bwd"] = {
        "workload": f"B={Bc} T={T} H={Ht} D={D}, forward (fused chunk kernel: y, boundary states, state_dot_a) and "
                    "backward (adjoint scan + chunk-parallel tensor-core backward)",
        "tokens_per_s": n_tok / sec, "ms": sec * 1e3, "tensor_frac_of_bf16_peak": n_tok * Ht * 294912 / sec / bf16,
        "gpu_launches_per_call": 3,
        "kernels": "wkv7_chunk_fused_kernel, wkv7_chunk_fused_kernel<adjoint>, wkv7_chunk_backward_kernel"}
    del toks, S0, dy
    torch.cuda.empty_cache()
    # ---- training forward + backward at head sizes 128 and 256 (serial CUDA-core recurrences; H * D = 4096)
    wide = {}
    Bw, Tw = 8, 1024
    cu_w, _ = synthetic.equal_length_metadata(Bw, Tw, device=dev)
    meta_w = make_chunk_metadata(cu_w, 64)
    for Dw in (128, 256):
        Hw = 4096 // Dw
        toks = [t.to(dev).requires_grad_() for t in synthetic.wkv7_inputs(Bw * Tw, Hw, Dw, seed=15)]
        S0 = synthetic.state_pool(Bw, Hw, Dw, seed=16, device=dev).requires_grad_()
        dy = torch.randn(Bw * Tw, Hw, Dw, device=dev).to(torch.bfloat16)

        def wide_step():
            res = F.statetune_recurrent_fp32io16(S0, *meta_w, *toks)
            res[0].backward(dy)
            for t in (*toks, S0):
                t.grad = None

        sec = _time_cuda(wide_step, warmup=1, iters=2)
        wide[f"D={Dw}"] = {"workload": f"B={Bw} T={Tw} H={Hw} D={Dw}", "tokens_per_s": Bw * Tw / sec, "ms": sec * 1e3}
        del toks, S0, dy
    out["training_fwd_bwd_wide_heads"] = wide
    torch.cuda.empty_cache()
    # ---- TMix layer chain, C = 2048
    C, Hh = 2048, 32
    g = torch.Generator().manual_seed(3)
    wt = lambda n, k: (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(dev)  # noqa: E731
    vec = lambda: torch.rand(C, generator=g).to(torch.bfloat16).to(dev)  # noqa: E731
    ranks = {"w": 96, "a": 96, "g": 256, "v": 64}
    # Four layers' weights (4 x 37.7 MB = 151 MB > the 126 MB L2), visited in turn: every layer streams its weights
    # from HBM as in a real model, instead of finding the one set of a single layer in L2 on every replay.
    n_layers = 4
    layers = [{"Wr": wt(C, C), "Wk": wt(C, C), "Wv": wt(C, C), "Wo": wt(C, C),
               "w1": {n: wt(r, C) for n, r in ranks.items()}, "w2": {n: wt(C, r) for n, r in ranks.items()}}
              for _ in range(n_layers)]
    mixes = [vec() for _ in range(6)]
    k_k, a0, k_a, r_k, lnw, lnb, v0 = (vec() for _ in range(7))
    for L in layers:
        L["packed"] = F.TMixLayerWeights(*mixes, L["Wr"], L["Wk"], L["Wv"], L["Wo"], L["w1"], L["w2"], k_k, a0, k_a, r_k,
                                         lnw, lnb, v0)
    weight_bytes = 2 * (4 * C * C + 2 * C * sum(ranks.values()))
    tmix = {}
    for M in (1, 4, 7, 512):
        x = torch.randn(M, C, generator=g).to(torch.bfloat16).to(dev)
        v_first = torch.randn(M, C, generator=g).to(torch.bfloat16).to(dev)
        shift = torch.zeros(M, C, dtype=torch.bfloat16, device=dev)
        spool = synthetic.state_pool(M, Hh, D, seed=5, device=dev)
        cu, idx = synthetic.equal_length_metadata(M, 1, device=dev)
        ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=M, state_pool_size=M, max_seqlen=1)

        def layer(L, fused=False):
            w1, w2 = L["w1"], L["w2"]
            if fused:  # token shift inside the projections: r, k, v and the four rank-in products in one launch
                r_, k_, v_, fw, fa, fg, fv = F.infer_tmix_shift_project_forward_varlen(
                    x, [mixes[0], mixes[2], mixes[3], mixes[1], mixes[4], mixes[5], mixes[3]],
                    [L["Wr"], L["Wk"], L["Wv"], w1["w"], w1["a"], w1["g"], w1["v"]], shift_state_pool=shift,
                    cu_seqlens=cu, state_indices=idx, max_seqlen=1, validated_metadata=ticket)
            else:      # the reference's operator sequence
                xr, xw, xk, xv, xa, xg = F.infer_tmix_mix6_forward_varlen(x, *mixes, shift_state_pool=shift,
                                                                          cu_seqlens=cu, state_indices=idx, max_seqlen=1,
                                                                          validated_metadata=ticket)
                r_ = F.infer_tmix_linear_forward_varlen(xr, L["Wr"])
                k_ = F.infer_tmix_linear_forward_varlen(xk, L["Wk"])
                v_ = F.infer_tmix_linear_forward_varlen(xv, L["Wv"])
                fw, fa, fg, fv = F.infer_tmix_lowrank_wagv_in_forward_varlen(xw, xa, xg, xv, w1["w"], w1["a"], w1["g"],
                                                                            w1["v"])
            w_, a12, g_, vres = F.infer_tmix_lowrank_vres_forward_varlen(fw, fa, fg, fv, w2["w"], w2["a"], w2["g"], w2["v"],
                                                                        v_, v_first, v0)
            kk_, nkk, kka = F.infer_tmix_kk_a_gate_forward_varlen(k_, k_k, a0, a12, k_a)
            sh = (M, Hh, D)
            y = F.infer_recurrent_fp32io16_forward_varlen(r_.view(sh), w_.view(sh), kk_.view(sh), vres.view(sh),
                                                          nkk.view(sh), kka.view(sh), state_pool=spool, cu_seqlens=cu,
                                                          state_indices=idx, validated_metadata=ticket, max_seqlen=1)
            z = F.infer_tmix_lnx_rkvres_xg_forward_varlen(y.view(M, C), r_, kk_, vres, r_k, lnw, lnb, g_)
            return F.infer_tmix_linear_forward_varlen(z, L["Wo"])

        def one_launch(L):  # the whole layer as one persistent kernel (decode batches of at most 8 rows)
            return F.infer_tmix_decode_layer_forward_varlen(x, v_first, L["packed"], shift_state_pool=shift,
                                                            state_pool=spool, cu_seqlens=cu, state_indices=idx,
                                                            validated_metadata=ticket)

        def stack(fused=False):
            for L in layers:
                if fused == "one_launch":
                    one_launch(L)
                else:
                    layer(L, fused)

        sec = _time_cuda(stack, warmup=3, iters=10) / n_layers
        # the same launches replayed from a CUDA graph: device time without the per-call host work
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        gsecs = {}
        with torch.cuda.stream(side):
            gticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=M, state_pool_size=M, max_seqlen=1)
            ticket = gticket
            for fused in (False, True) + (("one_launch",) if M <= 8 else ()):
                stack(fused)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    stack(fused)
                gsecs[fused] = _time_cuda(graph.replay, warmup=3, iters=30) / n_layers
                del graph
        torch.cuda.current_stream().wait_stream(side)
        gsec = gsecs[False]
        entry = {"us_per_layer": sec * 1e6, "us_per_layer_cuda_graph": gsec * 1e6, "gpu_launches_per_layer": 11,
                 "us_per_layer_fused_shift_cuda_graph": gsecs[True] * 1e6,
                 "gpu_launches_per_layer_fused_shift": 7 if M <= 8 else 10,
                 "l2": f"{n_layers} layers' weights ({n_layers * weight_bytes / 1e6:.0f} MB) visited in turn: larger than L2"}
        if M <= 7:
            entry["weight_hbm_frac_cuda_graph"] = weight_bytes / gsec / hbm
            entry["weight_hbm_frac_fused_shift_cuda_graph"] = weight_bytes / gsecs[True] / hbm
            entry["us_per_layer_one_launch_cuda_graph"] = gsecs["one_launch"] * 1e6
            entry["gpu_launches_per_layer_one_launch"] = 1
            entry["weight_hbm_frac_one_launch_cuda_graph"] = weight_bytes / gsecs["one_launch"] / hbm
        else:
            entry["tensor_frac_of_bf16_peak_cuda_graph"] = 2 * M * (4 * C * C + 2 * C * sum(ranks.values())) / gsec / bf16
        tmix[f"M={M}"] = entry
    out["tmix_layer_C2048"] = tmix
    del layers
    torch.cuda.empty_cache()
    out["tmix_train_glue"] = _extras_glue(dev, hbm)
    return out


class DecodeLoop:
    """The benchmark step on one rank: DECODE_STEPS_PER_STEP decode launches of `n_seq` sequences, replayed as one
    CUDA graph (or launched from Python), over one state pool or over several pools visited in turn."""

    def __init__(self, F, synthetic, dev, n_seq: int, seed: int, pools: int = 1, graph: bool = True, torch=None):
        self.n_seq = n_seq
        self.cu, self.idx = (t.to(dev) for t in synthetic.equal_length_metadata(n_seq, 1))
        self.pools = [synthetic.state_pool(n_seq, H, D, seed=seed + 31 * j, device=dev) for j in range(pools)]
        # each decode step's six token tensors live in one pinned host buffer [6, n_seq, H, D] (what a serving
        # host's staging area looks like); ring_host[i] are views of it
        self.ring_packed = [torch.stack(synthetic.wkv7_inputs(n_seq, H, D, seed=seed + 1 + i)).pin_memory()
                            for i in range(TOKEN_RING)]
        self.ring_host = [list(p.unbind(0)) for p in self.ring_packed]
        ring = [[t.to(dev) for t in step] for step in self.ring_host]
        self.ticket = F.prepare_recurrent_metadata(self.cu, self.idx, total_tokens=n_seq, state_pool_size=n_seq,
                                                   max_seqlen=1)
        self.kw = dict(cu_seqlens=self.cu, state_indices=self.idx, max_seqlen=1)

        def steps(ticket):
            for i in range(DECODE_STEPS_PER_STEP):
                F.infer_recurrent_fp32io16_forward_varlen(*ring[i % TOKEN_RING], state_pool=self.pools[i % pools],
                                                          validated_metadata=ticket, **self.kw)

        self.step = lambda: steps(self.ticket)
        self.launch_mode = f"{DECODE_STEPS_PER_STEP} Python launches per step"
        if graph:
            # every operator that takes a prepared ticket launches without host synchronisation, so the whole
            # step captures; a ticket is bound to the stream it was prepared on
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                g_ticket = F.prepare_recurrent_metadata(self.cu, self.idx, total_tokens=n_seq, state_pool_size=n_seq,
                                                        max_seqlen=1)
                F.infer_recurrent_fp32io16_forward_varlen(*ring[0], state_pool=self.pools[0],
                                                          validated_metadata=g_ticket, **self.kw)
                torch.cuda.synchronize(dev)
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph, stream=side):
                    steps(g_ticket)
            torch.cuda.current_stream(dev).wait_stream(side)
            self.step = self.graph.replay
            self.launch_mode = f"one CUDA graph of the {DECODE_STEPS_PER_STEP} decode launches per step"

    @property
    def bytes_per_launch(self) -> int:
        return self.n_seq * H * BYTES_PER_UNIT


def _profiled_traffic():
    """DRAM bytes per decode launch at the benchmark's full batch, from the ncu capture kept beside its summary."""
    p = ROOT / "profiles" / "wkv7_decode_pipelined_B256_H32.json"
    try:
        d = json.loads(p.read_text())
        return int(d["dram_bytes_per_launch"]), d.get("source", p.name)
    except Exception:
        return None, None


def run_b200(args):
    import torch
    import torch.distributed as dist

    import flashrwkv_b200 as F
    from flashrwkv_b200 import sharding, synthetic

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback of the product path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # the fixed batch of B sequences is split over the ranks: rank i owns a contiguous block and its state slots
    plan = sharding.shard_plan(B, H, world, rank)
    s0, s1 = plan["sequences"]
    n_local = s1 - s0
    loop = DecodeLoop(F, synthetic, dev, n_local, seed=20260805 + 1009 * rank, graph=not args.no_graph, torch=torch)

    # end to end: every decode step's six token tensors come from pinned host memory and its output goes back to
    # pinned host memory, through the package's three-stream host loop (copy-in / kernel / copy-out overlap)
    from flashrwkv_b200.host_io import HostDecodeLoop

    host_loop = HostDecodeLoop(loop.ring_host[0], state_pool=loop.pools[0], validated_metadata=loop.ticket, **loop.kw)
    y_hosts = [torch.empty((n_local, H, D), dtype=torch.bfloat16).pin_memory() for _ in range(4)]

    def e2e_step():
        for i in range(DECODE_STEPS_PER_STEP):
            host_loop.submit(loop.ring_packed[i % TOKEN_RING], y_hosts[i % len(y_hosts)])
        host_loop.drain()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, warmup, steps, sampler=None):
        for _ in range(warmup):
            fn()
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler:
            sampler.timed = True
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        barrier()
        if sampler:
            sampler.timed = False
        ms = start.elapsed_time(stop)
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else
                           int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank]))
    sampler.start()
    ms = timed(loop.step, args.warmup, args.steps, sampler)
    sampler.stop()
    e2e_steps = max(1, min(args.steps, 5))
    e2e_ms = timed(e2e_step, 1, e2e_steps) if not args.kernel_only else float("nan")

    tokens_per_step = B * DECODE_STEPS_PER_STEP  # the whole job: all ranks together decode the B sequences
    value = tokens_per_step * args.steps / (ms * 1e-3)
    e2e_value = tokens_per_step * e2e_steps / (e2e_ms * 1e-3)
    launches = args.steps * DECODE_STEPS_PER_STEP
    launch_s = ms * 1e-3 / launches
    peak, peak_kind = _peaks()
    achieved = loop.bytes_per_launch / launch_s / 1e9
    working_mb = n_local * H * D * D * 4 / 1e6
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_source": f"of {peak_kind}",
                # the library sends batches of at most 4608 (sequence, head) tiles to the register kernel
                "kernel": "wkv7_decode_pipelined_kernel" if n_local * H > 4608 else "wkv7_recurrent_d64_kernel",
                "algorithmic_bytes_per_launch": loop.bytes_per_launch, "us_per_launch": launch_s * 1e6,
                "note": "achieved = algorithmic bytes / time: an effective bandwidth that counts state tiles found in L2 "
                        "(the traversal order alternates between launches) as if they came from HBM"}
    extras_multi = {}
    if world == 1:
        traffic, source = _profiled_traffic()
        if traffic is not None:
            roofline["traffic"] = traffic
            roofline["traffic_source"] = source
            roofline["frac_dram"] = traffic / launch_s / 1e9 / peak
        if not args.kernel_only:
            # cold-L2 companion: two pools visited in turn (2 x 134 MB), so that no state tile of a launch is still
            # in the 126 MB L2 when its pool comes round again
            cold = DecodeLoop(F, synthetic, dev, n_local, seed=77, pools=2, graph=not args.no_graph, torch=torch)
            cold_ms = timed(cold.step, 2, max(2, args.steps // 4))
            cold_s = cold_ms * 1e-3 / (max(2, args.steps // 4) * DECODE_STEPS_PER_STEP)
            roofline["cold_l2"] = {"us_per_launch": cold_s * 1e6, "achieved": cold.bytes_per_launch / cold_s / 1e9,
                                   "frac": cold.bytes_per_launch / cold_s / 1e9 / peak,
                                   "how": "two state pools visited alternately: every tile comes from HBM"}
            del cold
    else:
        # the optional collective: all ranks' outputs of one decode step gathered on every rank (NCCL all-gather)
        y_local = torch.zeros((n_local, H, D), dtype=torch.bfloat16, device=dev)
        gather = lambda: sharding.gather_shards(y_local, plan, total=B)  # noqa: E731
        full = gather()
        reps = 20
        g_ms = timed(gather, 3, reps)
        extras_multi["gather_outputs"] = {"us": g_ms / reps * 1e3, "bytes_per_rank": y_local.numel() * 2,
                                          "gathered_shape": list(full.shape), "backend": "nccl all_gather",
                                          "note": "reported apart from the compute time; the data path has no collective"}
        if not args.kernel_only:
            # weak scaling beside it: every rank decodes a full batch of B sequences of its own
            weak = DecodeLoop(F, synthetic, dev, B, seed=555 + rank, graph=not args.no_graph, torch=torch)
            w_steps = max(2, args.steps // 4)
            w_ms = timed(weak.step, 2, w_steps)
            extras_multi["weak_scaling"] = {"tokens_per_s": B * world * DECODE_STEPS_PER_STEP * w_steps / (w_ms * 1e-3),
                                            "sequences_per_gpu": B, "global_sequences": B * world,
                                            "ms_per_step": w_ms / w_steps}
            del weak
            # chunked prefill (B=8 sequences of 4096 tokens, H=32) with the sequences split over the ranks
            from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata, wkv7_chunk_forward

            Bc, T, Hc = 8, 4096, 32
            cplan = sharding.shard_plan(Bc, Hc, world, rank)
            nb = cplan["sequences"][1] - cplan["sequences"][0]
            nh = cplan["heads"][1] - cplan["heads"][0]
            toks = [t.to(dev) for t in synthetic.wkv7_inputs(nb * T, nh, D, seed=11 + rank)]
            ccu, _ = synthetic.equal_length_metadata(nb, T, device=dev)
            meta = make_chunk_metadata(ccu, 64)
            cpool = synthetic.state_pool(nb, nh, D, seed=12, device=dev)
            c_ms = timed(lambda: wkv7_chunk_forward(*toks, state=cpool, chunk_metadata=meta), 2, 5)
            extras_multi["chunked_prefill"] = {"workload": f"B={Bc} T={T} H={Hc} split over {world} ranks by "
                                                           f"{cplan['axis']}: {nb} sequence(s) x {nh} heads per rank",
                                               "tokens_per_s": Bc * T * 5 / (c_ms * 1e-3), "ms": c_ms / 5}

    if rank == 0:
        cpu = _cpu_baseline(32) if world == 1 and not args.kernel_only else None
        l2_note = (f"no flush: the per-launch working set ({working_mb:.0f} MB of state) exceeds the 126 MB L2"
                   if working_mb > 126 else
                   f"the per-rank working set ({working_mb:.0f} MB of state) fits the 126 MB L2, so this split is bound "
                   f"by launch latency and L2, not by HBM")
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"recurrent decode B={B} H={H} D={D}, bf16 tokens, fp32 state, "
                                   f"{DECODE_STEPS_PER_STEP} consecutive decode steps per step",
                       "launch": loop.launch_mode, "global_sequences": B, "sequences_per_gpu": n_local,
                       "parallelism": f"the {B} sequences split over {world} GPU(s), no collective on the data path",
                       "l2": l2_note},
            "roofline": roofline,
            "e2e": {"value": e2e_value, "unit": "tokens/s",
                    "h2d_bytes_per_step": 6 * B * H * D * 2 * DECODE_STEPS_PER_STEP,
                    "d2h_bytes_per_step": B * H * D * 2 * DECODE_STEPS_PER_STEP, "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": sampler.summary(),
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if extras_multi:
            line["extras"] = extras_multi
        if world == 1 and not args.kernel_only and not args.no_extras:
            try:
                line["extras"] = _extras(dev)
            except Exception as exc:  # the headline line must survive a failure of the secondary workloads
                line["extras"] = {"error": f"{type(exc).__name__}: {exc}"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---- small workloads for profiler captures (python bench.py --profile-case NAME) -------------------------------
# Each holds well under a few GB on the device, uses inputs larger than the 126 MB L2 where DRAM figures matter,
# runs a handful of launches and exits, so that an `ncu` capture of one of its kernels ends by itself:
#   chunk      chunked forward, fused kernel: B=8, T=1024, H=32 (256 (sequence, head) pairs, 4096 (chunk, head) items)
#   chunk2k    chunked forward, build + scan kernels: B=2, T=4096, H=32 (4096 (chunk, head) items)
#   train      StateTune forward + backward: B=2, T=2048, H=32
#   train512   the same at B=8, T=512, H=64: 512 (sequence, head) pairs, as in the training configuration
#   tmix       one TMix layer's projections at C=2048 for M in (4, 512)
#   decode     recurrent decode steps at B=256, H=32 (the benchmark's shape, 8 launches)
#   decode32   the same at B=32: a rank's share of the batch at 8 GPUs (register kernel, tables not read)
#   decode16   the same on an fp16 state pool
#   glue       training-side TMix glue, forward + backward of the five operators: B=2, T=4096, C=4096
def _profile_case(name: str) -> None:
    import torch

    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata, wkv7_chunk_forward

    def case_chunk(reps: int = 3, B: int = 8, T: int = 1024, H: int = 32, path: int = 1):
        toks = [t.cuda() for t in synthetic.wkv7_inputs(B * T, H, D, seed=1)]
        cu, _ = synthetic.equal_length_metadata(B, T, device="cuda")
        pool = synthetic.state_pool(B, H, D, seed=2, device="cuda")
        meta = make_chunk_metadata(cu, 64)
        for _ in range(reps):
            wkv7_chunk_forward(*toks, state=pool, chunk_metadata=meta, path=path)

    def case_train(reps: int = 2, B: int = 2, T: int = 2048, H: int = 32):
        toks = [t.cuda().requires_grad_() for t in synthetic.wkv7_inputs(B * T, H, D, seed=3)]
        S0 = synthetic.state_pool(B, H, D, seed=4, device="cuda").requires_grad_()
        cu, _ = synthetic.equal_length_metadata(B, T, device="cuda")
        meta = make_chunk_metadata(cu, 64)
        dy = torch.randn(B * T, H, D, device="cuda").to(torch.bfloat16)
        for _ in range(reps):
            out = F.statetune_recurrent_fp32io16(S0, *meta, *toks)
            out[0].backward(dy)


    def case_tmix(reps: int = 3):
        C, H = 2048, 32
        g = torch.Generator().manual_seed(3)
        wt = lambda n, k: (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).cuda()  # noqa: E731
        ranks = {"w": 96, "a": 96, "g": 256, "v": 64}
        Wr = wt(C, C)
        w1 = {n: wt(r, C) for n, r in ranks.items()}
        w2 = {n: wt(C, r) for n, r in ranks.items()}
        v0 = torch.rand(C, generator=g).to(torch.bfloat16).cuda()
        for M in (4, 512):
            xs = [torch.randn(M, C, generator=g).to(torch.bfloat16).cuda() for _ in range(6)]
            for _ in range(reps):
                F.infer_tmix_linear_forward_varlen(xs[0], Wr)
                feats = F.infer_tmix_lowrank_wagv_in_forward_varlen(xs[1], xs[2], xs[3], xs[4], w1["w"], w1["a"], w1["g"],
                                                                    w1["v"])
                F.infer_tmix_lowrank_vres_forward_varlen(*feats, w2["w"], w2["a"], w2["g"], w2["v"], xs[4], xs[5], v0)


    def case_decode(reps: int = 8, B: int = B):
        cu, idx = synthetic.equal_length_metadata(B, 1, device="cuda")
        pool = synthetic.state_pool(B, H, D, seed=5, device="cuda")
        toks = [t.cuda() for t in synthetic.wkv7_inputs(B, H, D, seed=6)]
        ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=B, state_pool_size=B, max_seqlen=1)
        for _ in range(reps):
            F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool, cu_seqlens=cu, state_indices=idx,
                                                      validated_metadata=ticket, max_seqlen=1)


    def case_decode16(reps: int = 8):
        cu, idx = synthetic.equal_length_metadata(B, 1, device="cuda")
        pool = synthetic.state_pool(B, H, D, seed=5, device="cuda").half()
        elapsed = torch.zeros(B, dtype=torch.int32, device="cuda")
        toks = [t.cuda() for t in synthetic.wkv7_inputs(B, H, D, seed=6)]
        ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=B, state_pool_size=B, max_seqlen=1)
        for _ in range(reps):
            F.infer_recurrent_fp16_forward_varlen(*toks, state_pool=pool, elapsed_state_pool=elapsed, cu_seqlens=cu,
                                                  state_indices=idx, validated_metadata=ticket, max_seqlen=1)
            F.infer_recurrent_fp16_advance_i32(elapsed, 1)


    def case_glue(reps: int = 2):
        B, T, C = 2, 4096, 4096
        gen = torch.Generator(device="cuda").manual_seed(7)
        rn = lambda *s: torch.randn(*s, device="cuda", generator=gen).to(torch.bfloat16).requires_grad_()  # noqa: E731
        x, r, k, v, g = (rn(B, T, C) for _ in range(5))
        vecs = [rn(C) for _ in range(6)]
        r_k = rn(C // D, D)
        go = [torch.randn(B, T, C, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(6)]
        for _ in range(reps):
            outs = [F.pretrain_tmix_a_gate_bf16(vecs[0], x), F.pretrain_tmix_vres_gate_bf16(x, r, vecs[0], k),
                    *F.pretrain_tmix_kk_pre_bf16(x, vecs[0], r, vecs[1]),
                    F.pretrain_tmix_lnx_rkvres_xg_bf16(x, r, k, v, r_k, vecs[1], vecs[2], g)]
            torch.autograd.backward(outs, go[:len(outs)])
            torch.autograd.backward(F.pretrain_tmix_mix6_bf16(x, *vecs), go)

    def case_layer(reps: int = 3, M: int = 4):
        C = 2048
        g = torch.Generator().manual_seed(3)
        wt = lambda n, k: (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).cuda()  # noqa: E731
        vec = lambda: torch.rand(C, generator=g).to(torch.bfloat16).cuda()  # noqa: E731
        ranks = {"w": 96, "a": 96, "g": 256, "v": 64}
        layers = [F.TMixLayerWeights(vec(), vec(), vec(), vec(), vec(), vec(), wt(C, C), wt(C, C), wt(C, C), wt(C, C),
                                     {n: wt(r, C) for n, r in ranks.items()}, {n: wt(C, r) for n, r in ranks.items()},
                                     vec(), vec(), vec(), vec(), vec(), vec(), vec()) for _ in range(4)]
        x = torch.randn(M, C, generator=g).to(torch.bfloat16).cuda()
        v_first = torch.randn(M, C, generator=g).to(torch.bfloat16).cuda()
        shift = torch.zeros(M, C, dtype=torch.bfloat16, device="cuda")
        pool = synthetic.state_pool(M, C // D, D, seed=5, device="cuda")
        cu, idx = synthetic.equal_length_metadata(M, 1, device="cuda")
        ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=M, state_pool_size=M, max_seqlen=1)
        for _ in range(reps):
            for L in layers:  # four layers' weights in turn (151 MB): every launch streams its weights from HBM
                F.infer_tmix_decode_layer_forward_varlen(x, v_first, L, shift_state_pool=shift, state_pool=pool,
                                                         cu_seqlens=cu, state_indices=idx, validated_metadata=ticket)

    cases = {"layer": case_layer, "layer1": lambda: case_layer(3, 1), "chunk": case_chunk, "chunk2k": lambda: case_chunk(3, 2, 4096, 32, 0), "train": case_train,
             "train512": lambda: case_train(2, 8, 512, 64), "tmix": case_tmix, "decode": case_decode,
             "decode32": lambda: case_decode(8, 32),
             "decode16": case_decode16, "glue": case_glue}
    if name not in cases:
        raise SystemExit("unknown profile case; one of: " + ", ".join(sorted(cases)))
    cases[name]()
    torch.cuda.synchronize()
    print(f"profile case {name}: done")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("b200", "reference"), default="b200")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary workloads (prefill, training, TMix)")
    ap.add_argument("--no-graph", action="store_true", help="launch the decode steps from Python instead of one CUDA graph")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU-baseline legs (for profiler runs)")
    ap.add_argument("--profile-case", default=None, help="run one small workload for a profiler capture and exit")
    args = ap.parse_args()
    if args.profile_case:
        _profile_case(args.profile_case)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
