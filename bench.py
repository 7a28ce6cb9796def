#!/usr/bin/env python
"""Benchmark of the decoder hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--repeats R] [--impl b200|reference] [--workload ...]

Headline workload (BASELINE.json configs[1]): Llama-7B-shaped fp16 batch-1 greedy decode (32 layers, hidden 4096,
32 heads x 128, FFN 11008, vocab 32000), KV cache prefilled to 2048 tokens with N(0,1), random weights N(0,0.02);
one "step" = one generated token through executor.run().  Prints ONE JSON line (rank 0).

value  : tokens/s with token / position / cache state resident on the device (CUDA-graph replays only).  The timed
         block of K steps is repeated R times, every block bracketed by barrier + synchronise and timed with CUDA events;
         ms_per_step is the median block / K, and the line lists every block with the SM clock sampled in it.
e2e    : tokens/s when every step's input token comes from pinned host memory (H2D inside the timed region)
         and the sampled token is read back (D2H + synchronise) through the executor API.
roofline: the dominant kernel's algorithmic bytes per launch / its CUDA-event duration against the measured HBM copy
         peak (the one-kernel step itself; the weight-streaming linear kernel alone is timed next to it).
workloads / tensor_parallel (default workload only, same JSON line): the batch-32 paged decode and the bf16 prefill
         (one GPU), and the 70B-shaped grouped-query model — a 10-layer slice on one GPU, tensor-parallel over the N
         GPUs otherwise, with a parity check of the all-reduce and of a sharded decode step before its timed loop.
         With N > 1 `value` remains N independent replicas of the headline workload.
cpu_baseline / --impl reference: the reference's own CPU kernels (oracle/_ref, else the C port) on the host.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np

FALLBACK_HBM_GBS = 6650.0
FALLBACK_TFLOPS = 1400.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="7b", choices=["7b", "tiny", "7b-4l", "7b-b32", "70b-tp", "7b-prefill"],
                    help="7b: batch-1 greedy decode (the reported configuration; N > 1 = independent replicas). "
                         "7b-b32: batch 32, paged KV, top-k 50 sampling.  70b-tp: 70B-shaped GQA decode, tensor-parallel over N GPUs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--repeats", type=int, default=5,
                    help="the timed block of --steps steps is run this many times; ms_per_step is the median block / steps")
    ap.add_argument("--only-headline", action="store_true",
                    help="default workload only: skip the other configurations that are otherwise attached to the same JSON line")
    ap.add_argument("--graph", default="single", choices=["single", "fused"],
                    help="7b / tiny workloads: 'single' = the whole step as one persistent kernel (b200::DecodeStep); "
                         "'fused' = five fused launches per layer replayed as a CUDA graph")
    ap.add_argument("--case", default=None, choices=["linear_gate_up", "linear_down", "linear_qkv", "attn_decode", "attn_decode_b32", "attn_decode_gqa", "attn_decode_gqa_tp2", "topk", "gemm_qkv", "gemm_down", "gemm_gate_up",
                             "gemm_skinny16", "gemm_skinny32", "gemm_tp8", "all_reduce", "decode_step_timeline",
                             "rms_norm", "softmax", "gather", "attn_prefill", "skinny_qkv_tp8", "topk_sample"],
                    help="time one kernel alone at its 7B decode shape (small footprint; the case ncu captures run)")
    ap.add_argument("--launches", type=int, default=6)
    ap.add_argument("--shard-of", type=int, default=0,
                    help="with --workload 70b-tp on one GPU: run one rank's share of an N-way tensor-parallel step (all 80 layers, "
                         "the all-reduce left out). A diagnostic for launch lists; its line is marked and is not a benchmark value")
    return ap.parse_args()


def workload_config(name, world=1):
    from refactorgraph_b200.config import LlamaConfig      # pure Python: the reference arm must not load the kernel library
    if name == "tiny":  # for quick functional runs only; never the reported configuration
        return LlamaConfig(layers=2, hidden=512, heads=4, kv_heads=4, head_dim=128, ffn=1024, vocab=2000, max_seq=512), 256
    if name == "7b-4l":  # four 7B-shaped layers (2.3 GB on the device): the size ncu captures of the decode step use
        return LlamaConfig(layers=4, max_seq=2048 + 512), 2048
    if name == "7b-b32":
        return LlamaConfig(max_seq=4096 + 128, batch=32), 0
    if name == "70b-tp":
        # one GPU cannot hold 137 GB of weights next to the cache: a 10-layer slice, as the configuration states
        return LlamaConfig(layers=80 if world > 1 else 10, hidden=8192, heads=64, kv_heads=8, head_dim=128, ffn=28672,
                           vocab=32000, max_seq=4096 + 128, batch=16), 4096
    return LlamaConfig(max_seq=2048 + 512), 2048


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ----------------------------------------------------------------------------------------------------------
# CPU baseline: the reference's CPU kernels for one decoder layer (+ LM head) of one token, fp32, 1 core.
class CpuLayer:
    def __init__(self, cfg, kv_len):
        import oracle
        self.oracle = oracle
        self.kind = "reference" if oracle.load_ref() is not None else "port"
        rng = np.random.default_rng(0)
        H, D, nH, F = cfg.hidden, cfg.head_dim, cfg.heads, cfg.ffn
        self.cfg, self.L = cfg, kv_len
        f32 = lambda *s: (0.02 * rng.standard_normal(s, dtype=np.float32))
        self.x = rng.standard_normal((1, H), dtype=np.float32)
        self.g = np.ones(H, np.float32)
        self.wqkv, self.wo = f32(3 * nH * D, H), f32(H, nH * D)
        self.wg, self.wu, self.wd = f32(F, H), f32(F, H), f32(H, F)
        self.kc = rng.standard_normal((nH, kv_len, D), dtype=np.float32)
        self.vc = rng.standard_normal((nH, kv_len, D), dtype=np.float32)
        self.lm = None

    def _mm(self, a, b, trans_b=True):
        if self.kind == "reference":
            return self.oracle.ref_mat_mul(a, b, trans_b=trans_b)
        if a.ndim == 2:
            return self.oracle.port_mat_mul(a, b, trans_b=trans_b)
        return np.stack([self.oracle.port_mat_mul(a[i], b[i], trans_b=trans_b) for i in range(a.shape[0])])

    def layer(self):
        o, c = self.oracle, self.cfg
        ref = self.kind == "reference"
        rms = (lambda x: o.ref_rms_norm(x, self.g, c.eps)) if ref else (lambda x: o.port_rms_norm(x, self.g, c.eps))
        sm = (lambda s: o.ref_softmax(s, 2)) if ref else (lambda s: o.port_softmax_asbuilt(s, 2))
        n1 = rms(self.x)
        qkv = self._mm(n1, self.wqkv)                                        # weights stored [out, in]: transB
        q = np.ascontiguousarray(qkv[:, : c.heads * c.head_dim].reshape(c.heads, 1, c.head_dim))
        s = self._mm(q, self.kc)                                             # [nH, 1, L]
        p = sm(np.ascontiguousarray(s * np.float32(1.0 / np.sqrt(c.head_dim))))
        a = self._mm(p, self.vc, trans_b=False).reshape(1, c.heads * c.head_dim)
        h = self.x + self._mm(a, self.wo)
        n2 = rms(h)
        gt, up = self._mm(n2, self.wg), self._mm(n2, self.wu)
        act = gt * (1.0 / (1.0 + np.exp(-gt))) * up
        return h + self._mm(np.ascontiguousarray(act, dtype=np.float32), self.wd)

    def lm_head(self):
        if self.lm is None:
            self.lm = (0.02 * np.random.default_rng(1).standard_normal((self.cfg.vocab, self.cfg.hidden), dtype=np.float32))
        return self._mm(self.x, self.lm)


def cpu_baseline(cfg, kv_len, layer_reps=2):
    cl = CpuLayer(cfg, kv_len)
    cl.layer()  # warm caches / page in
    t0 = time.perf_counter()
    for _ in range(layer_reps):
        cl.layer()
    t_layer = (time.perf_counter() - t0) / layer_reps
    t0 = time.perf_counter()
    cl.lm_head()
    t_head = time.perf_counter() - t0
    tok_s = 1.0 / (cfg.layers * t_layer + t_head)
    return {"value": tok_s, "unit": "tokens/s", "cores": 1, "kind": cl.kind,
            "sample": f"{layer_reps} x one decoder layer for one token at KV {kv_len} ({t_layer:.3f} s each) + LM head once "
                      f"({t_head:.3f} s), fp32, weights stored [out,in] (transB); token time extrapolated x{cfg.layers} layers"}


def run_reference(args):
    """--impl reference: the reference's own CPU kernels on the host cores; each step = one decoder layer of one
    token (a bounded sample), tokens/s extrapolated over the layer count."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg, kv_len = workload_config(args.workload)
    cl = CpuLayer(cfg, kv_len)
    t0 = time.perf_counter()
    cl.lm_head()
    t_head = time.perf_counter() - t0
    for _ in range(max(1, min(args.warmup, 2))):
        cl.layer()
    steps = max(1, args.steps)
    budget_s = 150.0
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        cl.layer()
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    t_layer = (time.perf_counter() - t0) / done
    tok_s = 1.0 / (cfg.layers * t_layer + t_head)
    sample = (f"{done} timed steps, each one decoder layer of one token at KV {kv_len} ({t_layer:.3f} s) ; LM head timed once "
              f"({t_head:.3f} s); fp32; token time = {cfg.layers} x layer + head")
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 / tok_s, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(args.workload), "timed_steps_done": done},
            "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": 1, "kind": cl.kind, "sample": sample},
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_name(w):
    if w == "tiny":
        return "tiny functional decoder (not a reported configuration)"
    if w == "7b-4l":
        return "four Llama-7B-shaped layers + LM head, fp16 batch-1 greedy decode at KV 2048 (profiling size, not a reported configuration)"
    if w == "7b-b32":
        return "Llama-7B-shaped fp16 batch-32 decode, paged KV (16-token blocks), lengths uniform[512,4096], top-k 50 sampling"
    if w == "70b-tp":
        return "70B-shaped GQA fp16 batch-16 decode at KV 4096, tensor-parallel (column/row-sharded weights, all-reduce after O and down)"
    if w == "7b-prefill":
        return "Llama-7B-shaped bf16 prefill of 4 sequences x 2048 tokens (causal attention, KV cache written, first token by top-1)"
    return "Llama-7B-shaped fp16 batch-1 greedy decode, KV cache prefilled to 2048 tokens, one token per step"


# ----------------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi sampling during the timed region (read-only): SM clock, its maximum, power and the throttle reasons,
    every 50 ms, each sample with its wall-clock time so that it can be attributed to one timed block."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc, self.index = None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        """Returns (summary for the JSON line, [(unix time, sm MHz)] samples)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}, []
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        import datetime
        sm, mx, reasons, samples = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in out.strip().splitlines():
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            try:
                samples.append((datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp(), sm[-1]))
            except ValueError:
                pass
            for nm, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}, samples

    @staticmethod
    def window_mhz(samples, window):
        """Median SM clock of the samples taken inside [t0, t1]; the nearest sample when the window saw none."""
        if not samples:
            return None
        t0, t1 = window
        inside = [m for t, m in samples if t0 <= t <= t1]
        if inside:
            return statistics.median(inside)
        mid = 0.5 * (t0 + t1)
        return min(samples, key=lambda tm: abs(tm[0] - mid))[1]


def build_executor(cfg, kv_len, torch, workload="7b", world=1, rank=0, graph="single", shard_of=0):
    """Compiles the decode-step graph of the workload and fills weights and caches with seeded values generated on
    the device.  Returns (executor, index, state) where state holds what reset_state needs."""
    from refactorgraph_b200.llama import (decode_step_graph, decode_step_graph_batched, decode_step_graph_single_kernel, shard_config,
                                          weight_inputs)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(rank)
    dt = torch.float16
    state = {"lens0": np.full(cfg.batch, kv_len, np.int64), "paged": False}
    if workload in ("7b-b32", "70b-tp"):
        tp = world if workload == "70b-tp" else 1
        cfg = shard_config(cfg, shard_of if (shard_of and tp == 1) else tp)
        page = 16
        if workload == "7b-b32":
            lens0 = np.random.default_rng(0).integers(512, 4097, (cfg.batch,)).astype(np.int64)
            max_blocks = cfg.max_seq // page
            n_blocks = cfg.batch * max_blocks
            g, index = decode_step_graph_batched(cfg, paged=True, page=page, max_blocks=max_blocks, n_blocks=n_blocks,
                                                 top_k=50, sample=True, temperature=1.0, seed=0)
            state.update(lens0=lens0, paged=True, table=np.random.default_rng(1).permutation(n_blocks).reshape(cfg.batch, max_blocks).astype(np.int32))
            cache_shape = (n_blocks, cfg.kv_heads, page, cfg.head_dim)
        else:
            g, index = decode_step_graph_batched(cfg, world=tp)
            cache_shape = (cfg.batch, cfg.kv_heads, cfg.max_seq, cfg.head_dim)
        # the graphs are written operator by operator; the fusion pass turns the products and their readers into fused linear nodes
        passes = os.environ.get("RG_BENCH_PASSES", "fuse").split(",") if os.environ.get("RG_BENCH_PASSES", "fuse") else []
        ex = g.compiler().compile("cuda", "flat", passes)
        state["cfg"] = cfg
    else:
        g, index = decode_step_graph_single_kernel(cfg) if graph == "single" else decode_step_graph(cfg)
        ex = g.compiler().compile("cuda", "flat", [])
        cache_shape = (cfg.batch, cfg.kv_heads, cfg.max_seq, cfg.head_dim)
        state["cfg"] = cfg
    for name, shape in weight_inputs(cfg):
        w = torch.empty(shape, dtype=torch.float32, device="cuda").normal_(0.0, 0.02, generator=gen)
        if "norm" in name:
            w += 1.0
        w = w.to(dt)
        ex.set_input_blob(index[name], w.data_ptr(), w.numel() * 2)
        del w
    for l in range(cfg.layers):
        for nm in ("k_cache", "v_cache"):
            c = torch.empty(cache_shape, dtype=dt, device="cuda").normal_(0.0, 1.0, generator=gen)
            ex.set_input_blob(index[f"l{l}.{nm}"], c.data_ptr(), c.numel() * 2)
            del c
    if state["paged"]:
        ex.set_input(index["block_table"], state["table"])
    torch.cuda.empty_cache()
    return ex, index, state


def reset_state(ex, index, state, token0):
    ex.set_input(index["token"], token0)
    ex.set_input(index["pos"], state["lens0"])
    if "lens" in index:
        ex.set_input(index["lens"], state["lens0"] + 1)
    if "step" in index:
        ex.set_input(index["step"], np.zeros(1, np.int64))


def time_linear_kernel(ex, index, cfg, torch, stream, reps=3):
    """One pass over every linear launch of a step (real weights, eager launches on the executor's stream),
    bracketed by CUDA events: average launch duration and algorithmic bytes of the weight-streaming kernel."""
    from refactorgraph_b200 import capi
    B, H, D = cfg.batch, cfg.hidden, cfg.head_dim
    dt = torch.float16
    x = torch.randn(B, H, device="cuda").to(dt)
    act = torch.randn(B, cfg.ffn, device="cuda").to(dt)
    y = torch.empty(B, max(cfg.vocab, 2 * cfg.ffn), dtype=dt, device="cuda")
    gnorm = torch.ones(H, dtype=dt, device="cuda")
    calls, bytes_total = [], 0
    for l in range(cfg.layers):
        for name, n, k, src in ((f"l{l}.wqkv", (cfg.heads + 2 * cfg.kv_heads) * D, H, x), (f"l{l}.wo", H, cfg.heads * D, x),
                                (f"l{l}.wgu", 2 * cfg.ffn, H, x), (f"l{l}.wd", H, cfg.ffn, act)):
            p = capi.LinearParams()
            p.dtype, p.m, p.n, p.k = capi.FP16, B, n, k
            p.prologue, p.epilogue, p.epsilon = (1 if k == H and n != H else 0), (2 if "wgu" in name else 0), cfg.eps
            calls.append((p, [src.data_ptr(), ex.input_address(index[name]), gnorm.data_ptr() if p.prologue else 0, 0, 0, 0]))
            bytes_total += n * k * 2
    p = capi.LinearParams()
    p.dtype, p.m, p.n, p.k, p.prologue, p.epsilon = capi.FP16, B, cfg.vocab, H, 1, cfg.eps
    calls.append((p, [x.data_ptr(), ex.input_address(index["lm_head"]), gnorm.data_ptr(), 0, 0, 0]))
    bytes_total += cfg.vocab * H * 2
    sid = stream.cuda_stream
    outs = [y.data_ptr(), 0, 0]

    def one_pass():
        for p, ins in calls:
            capi.call("linear", p, ins, outs, stream=sid)
    one_pass()
    stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        one_pass()
    e1.record(stream)
    stream.synchronize()
    ms = e0.elapsed_time(e1) / reps
    return {"launches": len(calls), "ms_per_pass": ms, "bytes_per_pass": bytes_total,
            "avg_launch_us": 1000.0 * ms / len(calls), "gbs": bytes_total / (ms * 1e-3) / 1e9}


def time_paged_attention(cfg, lens_h, torch, stream, launches=20):
    """The attention launch of the paged batch workload alone (the kernel with the largest share of that step): the workload's
    own sequence lengths, 16-token pages in a shuffled block table, two cache pairs in rotation (each larger than L2)."""
    from refactorgraph_b200 import capi
    B, nH, D, page = cfg.batch, cfg.heads, cfg.head_dim, 16
    MS = 4096 + 128
    max_blocks = MS // page
    n_blocks = B * max_blocks
    dev = "cuda"
    table = torch.from_numpy(np.random.default_rng(1).permutation(n_blocks).reshape(B, max_blocks).astype(np.int32)).to(dev)
    q = torch.randn(B, nH, D, device=dev).to(torch.float16)
    caches = [(torch.randn(n_blocks, cfg.kv_heads, page, D, device=dev).to(torch.float16),
               torch.randn(n_blocks, cfg.kv_heads, page, D, device=dev).to(torch.float16)) for _ in range(2)]
    lens = torch.from_numpy(np.asarray(lens_h, dtype=np.int64)).to(dev)
    o = torch.empty_like(q)
    p = capi.AttnDecodeParams(capi.FP16, B, nH, MS, capi.KvLayout(cfg.kv_heads, D, MS, page, max_blocks))
    wsb = torch.zeros(capi.workspace("attn_decode", p), dtype=torch.uint8, device=dev)
    bytes_per = 2 * cfg.kv_heads * int(np.asarray(lens_h).sum()) * D * 2
    sid = stream.cuda_stream

    def launch(i):
        kc, vc = caches[i % 2]
        capi.call("attn_decode", p, [q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens.data_ptr(), table.data_ptr()], [o.data_ptr()],
                  ws=wsb.data_ptr(), stream=sid)
    for i in range(3):
        launch(i)
    stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(launches):
        launch(i)
    e1.record(stream)
    stream.synchronize()
    ms = e0.elapsed_time(e1) / launches
    return {"launches": launches, "avg_launch_us": 1000.0 * ms, "bytes_per_launch": bytes_per, "gbs": bytes_per / (ms * 1e-3) / 1e9}


def run_decode_step_timeline():
    """Per-phase timeline of the single-kernel decode step at the 7B shape (KV 2048), read back from the kernel's own
    %globaltimer stamps (rg_b200_decode_step_timeline)."""
    import ctypes as C
    import torch
    from refactorgraph_b200 import capi
    lib = capi.load()
    torch.cuda.set_device(0)
    torch.manual_seed(0)
    dt, dev = torch.float16, "cuda"
    L, H, nH, D, F, V, MS, pos0 = 32, 4096, 32, 128, 11008, 32000, 2560, 2048
    p = capi.DecodeStepParams(capi.FP16, L, H, nH, nH, D, F, V, MS, 1e-6, 10000.0)
    ws = torch.zeros(capi.workspace("decode_step", p), dtype=torch.uint8, device=dev)
    rnd = lambda *s: (torch.randn(*s, device=dev) * 0.02).to(dt)
    ones = lambda n: torch.ones(n, dtype=dt, device=dev)
    tok, pos = torch.tensor([5], device=dev), torch.tensor([pos0], device=dev)
    ins = [tok, pos, rnd(V, H), ones(H), rnd(V, H)]
    for _ in range(L):
        ins += [ones(H), rnd(3 * H, H), rnd(H, H), ones(H), rnd(2 * F, H), rnd(H, F),
                torch.randn(1, nH, MS, D, device=dev).to(dt), torch.randn(1, nH, MS, D, device=dev).to(dt)]
    outs = [torch.zeros(1, dtype=torch.int64, device=dev), torch.zeros(1, device=dev), torch.zeros(1, V, dtype=dt, device=dev)]
    torch.cuda.synchronize()
    for _ in range(4):
        capi.call("decode_step", p, [t.data_ptr() for t in ins], [t.data_ptr() for t in outs], ws=ws.data_ptr())
    torch.cuda.synchronize()
    n_entries = (5 * L + 2) * 4
    buf = (C.c_uint64 * n_entries)()
    n = lib.rg_b200_decode_step_timeline(C.byref(p), ws.data_ptr(), buf, n_entries)
    tt = np.array(buf[:n], dtype=np.float64).reshape(-1, 4)
    sub = np.zeros((5 * L + 1, 4))
    for ph in range(5 * L + 1):
        e, xr, ud, ep = tt[ph]
        nxt = tt[ph + 1, 0]
        sub[ph] = [(xr - e) / 1e3, (ud - xr) / 1e3, (ep - ud) / 1e3, (nxt - ep) / 1e3]
    names = ["qkv", "attention", "o", "gate_up", "down"]
    nbytes = [3 * H * H * 2, 2 * nH * pos0 * D * 2, H * H * 2, 2 * F * H * 2, F * H * 2]
    out = {"case": "decode_step_timeline", "total_us": (tt[5 * L + 1, 0] - tt[0, 0]) / 1e3, "error_state": lib.rg_b200_error_state(),
           "columns": ["x_ready_us", "units_us", "epilogue_us", "barrier_us", "phase_us", "GB/s"], "phases": {}}
    for k, nm in enumerate(names):
        m = sub[k:5 * L:5].mean(0)
        out["phases"][nm] = [round(float(v), 2) for v in m] + [round(float(m.sum()), 2), round(nbytes[k] / m.sum() / 1e3)]
    m = sub[5 * L]
    out["phases"]["lm_head"] = [round(float(v), 2) for v in m] + [round(float(m.sum()), 2), round(V * H * 2 / m.sum() / 1e3)]
    print(json.dumps(out), flush=True)


def run_all_reduce_case(args, torch, dist, rank, world):
    """The all-reduce of the tensor-parallel step alone (16 tokens x 8192, fp16, residual add fused), `--launches` calls
    back to back on every rank: device time per call, max over ranks."""
    from refactorgraph_b200 import capi
    count = 16 * 8192

    def exchange(handle):
        out = [None] * world
        dist.all_gather_object(out, handle)
        return out
    comm = capi.Comm(world, rank, count * 2, exchange=exchange if world > 1 else None)
    x = torch.randn(count, device="cuda").to(torch.float16)
    r = torch.randn(count, device="cuda").to(torch.float16)
    y = torch.empty_like(x)
    sid = torch.cuda.current_stream().cuda_stream
    for _ in range(5):
        comm.all_reduce(capi.FP16, 0, count, x.data_ptr(), y.data_ptr(), r.data_ptr(), stream=sid)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.launches):
        comm.all_reduce(capi.FP16, 0, count, x.data_ptr(), y.data_ptr(), r.data_ptr(), stream=sid)
    e1.record()
    torch.cuda.synchronize()
    us = torch.tensor([1000.0 * e0.elapsed_time(e1) / args.launches], device="cuda")
    if world > 1:
        dist.all_reduce(us, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"case": "all_reduce", "n_gpus": world, "count": count, "launches": args.launches, "us_per_call": round(float(us.item()), 2),
                          "comm_status": comm.status()}), flush=True)
    if world > 1:
        dist.barrier()
    comm.destroy()


def run_gemm_tp8(args):
    """The four matrix products one rank runs per layer of the 70B-shaped model at tensor-parallel 8 (16 tokens, fp16),
    each timed alone over weight buffers that together exceed L2."""
    import torch
    from refactorgraph_b200 import capi
    torch.cuda.set_device(0)
    capi.load()
    dev, dt, m = "cuda", torch.float16, 16
    sid = torch.cuda.current_stream().cuda_stream
    out = {"case": "gemm_tp8", "launches": args.launches, "products": {}}
    for name, n, k in (("qkv", 1280, 8192), ("o", 8192, 1024), ("gate_up", 7168, 8192), ("down", 8192, 3584)):
        nb = max(2, int(400e6 // (n * k * 2)))
        As = [torch.randn(m, k, device=dev).to(dt) for _ in range(2)]
        Bs = [(0.02 * torch.randn(n, k, device=dev)).to(dt) for _ in range(nb)]
        y = torch.empty(m, n, dtype=dt, device=dev)
        p = capi.MatMulParams()
        p.dtype, p.m, p.n, p.k, p.trans_b, p.alpha, p.beta, p.batch, p.stride_y, p.force_kernel = capi.FP16, m, n, k, 1, 1.0, 0.0, 1, m * n, 0
        p.flags = 0 if os.environ.get("RG_BENCH_NO_STATIC") else capi.MM_B_STATIC      # B is a weight, as in the decode graph
        nws = capi.workspace("mat_mul", p)
        wsb = torch.zeros(max(nws, 1), dtype=torch.uint8, device=dev)

        def launch(i):
            capi.call("mat_mul", p, [As[i % 2].data_ptr(), Bs[i % nb].data_ptr(), 0], [y.data_ptr()], ws=wsb.data_ptr() if nws else 0, stream=sid)
        for i in range(3):
            launch(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.launches):
            launch(i)
        e1.record()
        torch.cuda.synchronize()
        us = 1000.0 * e0.elapsed_time(e1) / args.launches
        out["products"][name] = {"n": n, "k": k, "us": round(us, 2), "gbs": round(n * k * 2 / us / 1e3)}
    print(json.dumps(out), flush=True)


def run_case(args):
    """One kernel alone at its Llama-7B decode shape, inputs rotated over buffers larger than L2 in total."""
    import torch
    from refactorgraph_b200 import capi
    if args.case == "decode_step_timeline":
        return run_decode_step_timeline()
    if args.case == "gemm_tp8":
        return run_gemm_tp8(args)
    torch.cuda.set_device(0)
    capi.load()
    dt, dev = torch.float16, "cuda"
    H, nH, D, F, V = 4096, 32, 128, 11008, 32000
    st = torch.cuda.current_stream()
    sid = st.cuda_stream
    nbuf = 4
    if args.case.startswith("linear"):
        n, k, pro, epi = {"linear_gate_up": (2 * F, H, 1, 2), "linear_down": (H, F, 0, 1), "linear_qkv": (3 * H, H, 1, 3)}[args.case]
        ws = [(0.02 * torch.randn(n, k, device=dev)).to(dt) for _ in range(nbuf)]
        x = torch.randn(1, k, device=dev).to(dt)
        g = torch.ones(k, dtype=dt, device=dev)
        r = torch.randn(1, n, device=dev).to(dt)
        y = torch.empty(1, n, dtype=dt, device=dev)
        kc = torch.zeros(1, nH, 256, D, dtype=dt, device=dev)
        vc = torch.zeros_like(kc)
        pos = torch.tensor([100], device=dev)
        p = capi.LinearParams()
        p.dtype, p.m, p.n, p.k, p.prologue, p.epilogue, p.epsilon, p.n_heads, p.theta = capi.FP16, 1, n, k, pro, epi, 1e-6, nH, 10000.0
        p.kv = capi.KvLayout(nH, D, 256, 0, 0)
        bytes_per = n * k * 2

        def launch(i):
            capi.call("linear", p, [x.data_ptr(), ws[i % nbuf].data_ptr(), g.data_ptr() if pro else 0, r.data_ptr() if epi == 1 else 0,
                                    pos.data_ptr() if epi == 3 else 0, 0], [y.data_ptr(), kc.data_ptr() if epi == 3 else 0, vc.data_ptr() if epi == 3 else 0], stream=sid)
    elif args.case.startswith("gemm"):
        bf = torch.bfloat16
        m, n, k = {"gemm_qkv": (8192, 3 * H, H), "gemm_down": (8192, H, F), "gemm_gate_up": (8192, 2 * F, H),
                   "gemm_skinny16": (16, 2 * F, H), "gemm_skinny32": (32, 2 * F, H)}[args.case]
        nb = 2 if m > 64 else nbuf
        As = [torch.randn(m, k, device=dev).to(bf) for _ in range(nb)]
        Bs = [(0.02 * torch.randn(n, k, device=dev)).to(bf) for _ in range(nb)]
        y = torch.empty(m, n, dtype=bf, device=dev)
        p = capi.MatMulParams()
        p.dtype, p.m, p.n, p.k, p.trans_b, p.alpha, p.beta, p.batch, p.stride_y, p.force_kernel = capi.BF16, m, n, k, 1, 1.0, 1.0, 1, m * n, 3
        bytes_per = (m * k + n * k + m * n) * 2
        flops_per = 2.0 * m * n * k
        nws = capi.workspace("mat_mul", p)
        wsb = torch.zeros(max(nws, 1), dtype=torch.uint8, device=dev)

        def launch(i):
            capi.call("mat_mul", p, [As[i % nb].data_ptr(), Bs[i % nb].data_ptr(), 0], [y.data_ptr()], ws=wsb.data_ptr() if nws else 0, stream=sid)
    elif args.case == "attn_decode":
        L, MS = 2112, 2560
        q = torch.randn(1, nH, D, device=dev).to(dt)
        caches = [(torch.randn(1, nH, MS, D, device=dev).to(dt), torch.randn(1, nH, MS, D, device=dev).to(dt)) for _ in range(nbuf * 2)]
        lens = torch.tensor([L], device=dev)
        o = torch.empty_like(q)
        p = capi.AttnDecodeParams(capi.FP16, 1, nH, MS, capi.KvLayout(nH, D, MS, 0, 0))
        wsb = torch.zeros(capi.workspace("attn_decode", p), dtype=torch.uint8, device=dev)
        bytes_per = 2 * nH * L * D * 2

        def launch(i):
            kc, vc = caches[i % len(caches)]
            capi.call("attn_decode", p, [q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens.data_ptr(), 0], [o.data_ptr()], ws=wsb.data_ptr(), stream=sid)
    elif args.case == "attn_decode_b32":
        # the attention launch of the batch-32 workload: 32 sequences, lengths uniform[512, 4096], 16-token pages
        B, page, MS = 32, 16, 4096 + 128
        lens_h = np.random.default_rng(0).integers(512, 4097, (B,)).astype(np.int64)
        max_blocks = MS // page
        n_blocks = B * max_blocks
        table = torch.from_numpy(np.random.default_rng(1).permutation(n_blocks).reshape(B, max_blocks).astype(np.int32)).to(dev)
        q = torch.randn(B, nH, D, device=dev).to(dt)
        caches = [(torch.randn(n_blocks, nH, page, D, device=dev).to(dt), torch.randn(n_blocks, nH, page, D, device=dev).to(dt)) for _ in range(2)]
        lens = torch.from_numpy(lens_h).to(dev)
        o = torch.empty_like(q)
        p = capi.AttnDecodeParams(capi.FP16, B, nH, MS, capi.KvLayout(nH, D, MS, page, max_blocks))
        wsb = torch.zeros(capi.workspace("attn_decode", p), dtype=torch.uint8, device=dev)
        bytes_per = 2 * nH * int(lens_h.sum()) * D * 2

        def launch(i):
            kc, vc = caches[i % len(caches)]
            capi.call("attn_decode", p, [q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens.data_ptr(), table.data_ptr()], [o.data_ptr()], ws=wsb.data_ptr(), stream=sid)
    elif args.case in ("attn_decode_gqa", "attn_decode_gqa_tp2"):
        # one rank's attention launch of the 70B-shaped model at tensor-parallel 8 (or 2): 16 sequences x 4096 tokens, 8 query
        # heads on 1 KV head (32 on 4)
        B, L, MS, nq, nkv = (16, 4096, 4096 + 128, 8, 1) if args.case == "attn_decode_gqa" else (16, 4096, 4096 + 128, 32, 4)
        q = torch.randn(B, nq, D, device=dev).to(dt)
        caches = [(torch.randn(B, nkv, MS, D, device=dev).to(dt), torch.randn(B, nkv, MS, D, device=dev).to(dt)) for _ in range(8)]
        lens = torch.full((B,), L, device=dev, dtype=torch.int64)
        o = torch.empty_like(q)
        p = capi.AttnDecodeParams(capi.FP16, B, nq, MS, capi.KvLayout(nkv, D, MS, 0, 0))
        wsb = torch.zeros(capi.workspace("attn_decode", p), dtype=torch.uint8, device=dev)
        bytes_per = 2 * nkv * B * L * D * 2

        def launch(i):
            kc, vc = caches[i % len(caches)]
            capi.call("attn_decode", p, [q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens.data_ptr(), 0], [o.data_ptr()], ws=wsb.data_ptr(), stream=sid)
    elif args.case == "rms_norm":
        # the prefill shape: 8192 tokens x 4096, bf16 (64 MiB in, 64 MiB out per launch; two buffers > L2)
        from refactorgraph_b200 import torch_ops as tops
        rows, dim = 8192, H
        xs = [torch.randn(rows, dim, device=dev).to(torch.bfloat16) for _ in range(3)]
        w = torch.ones(dim, dtype=torch.bfloat16, device=dev)
        y = torch.empty_like(xs[0])
        p = capi.RmsNormParams(capi.BF16, rows, dim, 1e-6, 0)
        bytes_per = 2 * rows * dim * 2

        def launch(i):
            capi.call("rms_norm", p, [xs[i % 3].data_ptr(), w.data_ptr()], [y.data_ptr()], stream=sid)
    elif args.case == "softmax":
        # attention-score shaped: [4 * 32 * 2048 rows, 2048] would be 1 GiB; a quarter of it (one sequence), fp16
        rows, n = 32 * 2048, 2048
        xs = [torch.randn(rows, n, device=dev).to(dt) for _ in range(2)]
        y = torch.empty_like(xs[0])
        p = capi.SoftmaxParams(capi.FP16, rows, n, 1)
        bytes_per = 2 * rows * n * 2

        def launch(i):
            capi.call("softmax", p, [xs[i % 2].data_ptr()], [y.data_ptr()], stream=sid)
    elif args.case == "gather":
        # embedding lookup of a prefill: 8192 token ids into a [32000, 4096] fp16 table
        table = torch.randn(V, H, device=dev).to(dt)
        ids = [torch.randint(0, V, (8192,), device=dev) for _ in range(4)]
        y = torch.empty(8192, H, dtype=dt, device=dev)
        p = capi.GatherParams(1, V, 8192, H * 2, capi.I64)
        bytes_per = 2 * 8192 * H * 2

        def launch(i):
            capi.call("gather", p, [table.data_ptr(), ids[i % 4].data_ptr()], [y.data_ptr()], stream=sid)
    elif args.case == "attn_prefill":
        # the attention launch of the prefill workload: [4, 32 heads, 2048 tokens, 128], bf16, causal; flops = 4 S^2 D / 2 per head
        bf, S = torch.bfloat16, 2048
        NB = int(os.environ.get("RG_BENCH_ATTN_SEQS", "4"))   # sequences per launch (the prefill workload has 4)
        qkv = [tuple(torch.randn(NB, nH, S, D, device=dev).to(bf) for _ in range(3)) for _ in range(2)]
        o = torch.empty(NB, nH, S, D, dtype=bf, device=dev)
        p = capi.AttentionParams(capi.BF16, NB, nH, nH, S, D, S, 0)
        bytes_per = 4 * NB * nH * S * D * 2
        flops_per = NB * nH * 4.0 * D * (S * (S + 1) / 2.0)

        def launch(i):
            q, k, v = qkv[i % 2]
            capi.call("attention", p, [q.data_ptr(), k.data_ptr(), v.data_ptr(), 0, 0, 0], [o.data_ptr(), 0, 0], stream=sid)
    elif args.case == "skinny_qkv_tp8":
        # one rank's QKV projection at tensor-parallel 8 (16 tokens, 1280 x 8192 weights) with the RoPE + cache-append epilogue
        m, nq, nkv, k, MS = 16, 8, 1, 8192, 4096 + 128
        n = (nq + 2 * nkv) * D
        ws_ = [(0.02 * torch.randn(n, k, device=dev)).to(dt) for _ in range(8)]
        x = torch.randn(m, k, device=dev).to(dt)
        y = torch.empty(m, nq * D, dtype=dt, device=dev)
        kc = torch.zeros(m, nkv, MS, D, dtype=dt, device=dev)
        vc = torch.zeros_like(kc)
        pos = torch.full((m,), 4096, device=dev, dtype=torch.int64)
        p = capi.LinearParams()
        p.dtype, p.m, p.n, p.k, p.prologue, p.epilogue, p.n_heads, p.theta = capi.FP16, m, n, k, 0, 3, nq, 10000.0
        p.kv = capi.KvLayout(nkv, D, MS, 0, 0, 0)
        wsb = torch.zeros(max(capi.workspace("linear", p), 1), dtype=torch.uint8, device=dev)
        bytes_per = n * k * 2

        def launch(i):
            capi.call("linear", p, [x.data_ptr(), ws_[i % 8].data_ptr(), 0, 0, pos.data_ptr(), 0], [y.data_ptr(), kc.data_ptr(), vc.data_ptr()],
                      ws=wsb.data_ptr(), stream=sid)
    elif args.case == "topk_sample":
        xs = [torch.randn(32, V, device=dev).to(dt) for _ in range(nbuf)]
        tok = torch.empty(32, dtype=torch.int64, device=dev)
        stp = torch.zeros(1, dtype=torch.int64, device=dev)
        p = capi.TopkSampleParams(capi.FP16, 32, V, 50, 1.0, 0)
        bytes_per = 32 * V * 2

        def launch(i):
            capi.call("topk_sample", p, [xs[i % nbuf].data_ptr(), stp.data_ptr()], [tok.data_ptr()], stream=sid)
    else:
        xs = [torch.randn(1, V, device=dev).to(dt) for _ in range(nbuf)]
        vals = torch.empty(1, 1, dtype=torch.float32, device=dev)
        idx = torch.empty(1, 1, dtype=torch.int64, device=dev)
        p = capi.TopkParams(capi.FP16, 1, V, 1, 1)
        bytes_per = V * 2

        def launch(i):
            capi.call("topk", p, [xs[i % nbuf].data_ptr()], [vals.data_ptr(), idx.data_ptr()], stream=sid)
    for i in range(3):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.launches):
        launch(i)
    e1.record()
    torch.cuda.synchronize()
    us = 1000.0 * e0.elapsed_time(e1) / args.launches
    out = {"case": args.case, "launches": args.launches, "us_per_launch": us, "algorithmic_bytes_per_launch": bytes_per,
           "gbs": bytes_per / us / 1e3}
    if args.case.startswith("gemm") or args.case == "attn_prefill":
        out["tflops"] = flops_per / us / 1e6
    print(json.dumps(out), flush=True)


def time_skinny_gemm(ex, index, cfg, torch, stream, reps=3):
    """Batched workloads: one pass over every weight MatMul of a step through rg_b200_mat_mul (tensor-core kernel with
    the skinny activation on the N side) on the real per-rank weights, bracketed by CUDA events."""
    from refactorgraph_b200 import capi
    B, H, D = cfg.batch, cfg.hidden, cfg.head_dim
    dt = torch.float16
    x = torch.randn(B, max(H, cfg.ffn, cfg.heads * D), device="cuda").to(dt)
    y = torch.empty(B, max(cfg.vocab, 2 * cfg.ffn), dtype=dt, device="cuda")
    calls, bytes_total = [], 0
    shapes = []
    for l in range(cfg.layers):
        shapes += [(f"l{l}.wqkv", (cfg.heads + 2 * cfg.kv_heads) * D, H), (f"l{l}.wo", H, cfg.heads * D),
                   (f"l{l}.wgu", 2 * cfg.ffn, H), (f"l{l}.wd", H, cfg.ffn)]
    shapes.append(("lm_head", cfg.vocab, H))
    for name, n, k in shapes:
        p = capi.MatMulParams()
        p.dtype, p.m, p.n, p.k, p.trans_b, p.alpha, p.beta, p.batch, p.stride_y = capi.FP16, B, n, k, 1, 1.0, 1.0, 1, B * n
        xk = x[:, :k].contiguous() if k != x.shape[1] else x
        nws = capi.workspace("mat_mul", p)
        wsb = torch.zeros(max(nws, 1), dtype=torch.uint8, device="cuda")
        calls.append((p, [xk.data_ptr(), ex.input_address(index[name]), 0], xk, wsb, nws))
        bytes_total += n * k * 2
    sid = stream.cuda_stream
    outs = [y.data_ptr()]
    torch.cuda.synchronize()

    def one_pass():
        for p, ins, _keep, wsb, nws in calls:
            capi.call("mat_mul", p, ins, outs, ws=wsb.data_ptr() if nws else 0, stream=sid)
    one_pass()
    stream.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        one_pass()
    e1.record(stream)
    stream.synchronize()
    ms = e0.elapsed_time(e1) / reps
    return {"launches": len(calls), "ms_per_pass": ms, "bytes_per_pass": bytes_total,
            "avg_launch_us": 1000.0 * ms / len(calls), "gbs": bytes_total / (ms * 1e-3) / 1e9}


def _barrier(torch, dist, world):
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def _max_over_ranks(torch, dist, world, values):
    if world == 1:
        return [float(v) for v in values]
    t = torch.tensor(list(values), device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def timed_blocks(torch, dist, world, stream, sampler, repeats, before_block, run_block):
    """`repeats` timed blocks; each block is bracketed by barrier + synchronize on both sides and timed with CUDA events on
    the executor's stream.  Returns per-block milliseconds (max over ranks) and the wall-clock window of every block (for
    binning the clock samples)."""
    ms, windows = [], []
    for _ in range(repeats):
        before_block()
        _barrier(torch, dist, world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        e0.record(stream)
        run_block()
        e1.record(stream)
        stream.synchronize()
        w1 = time.time()
        _barrier(torch, dist, world)
        ms.append(e0.elapsed_time(e1))
        windows.append((w0, w1))
    ms = _max_over_ranks(torch, dist, world, ms)
    return ms, windows


def block_summary(ms_blocks, windows, steps, sampler_samples):
    """Median block and what the others looked like: per-repeat ms/step, spread, SM clock seen in each window."""
    per_step = [m / steps for m in ms_blocks]
    med = statistics.median(per_step)
    mhz = [ClockSampler.window_mhz(sampler_samples, w) for w in windows]
    return med, {"repeats": len(ms_blocks), "repeat_ms_per_step": [round(v, 5) for v in per_step],
                 "repeat_spread": round((max(per_step) - min(per_step)) / med, 5) if med else None,
                 "repeat_sm_mhz": mhz,
                 "repeat_ms_times_mhz": [round(v * m, 2) if m else None for v, m in zip(per_step, mhz)]}


def tensor_peak():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"]), "measured sustained"
    except Exception:
        return FALLBACK_TFLOPS, "fallback"


def ncu_traffic_ratio(name):
    """DRAM bytes (read + written) per algorithmic byte from the tracked ncu summary of a kernel (profiles/<name>.json,
    written next to the text summary of the same capture); None when there is no such record."""
    try:
        rec = json.load(open(os.path.join(ROOT, "profiles", name + ".json")))
        return (float(rec["dram_bytes_read"]) + float(rec["dram_bytes_write"])) / float(rec["algorithmic_bytes"])
    except Exception:
        return None


def measure_prefill(args, torch, dist, lib, rank, world, local, steps, warmup, repeats):
    """BASELINE configuration 4: 7B-shaped bf16 prefill, batch 4 x 2048 tokens, causal; one step = one prefill of all
    8192 tokens (replicated per GPU when N > 1).  Tensor-bound: flops / time against the measured bf16 matmul peak."""
    from refactorgraph_b200.graph_builder import BF16
    from refactorgraph_b200.llama import LlamaConfig, prefill_graph, weight_inputs
    B, S = 4, 2048
    cfg = LlamaConfig(max_seq=S, batch=B, dtype=BF16)
    g, index = prefill_graph(cfg, S, fused_rope=not os.environ.get("RG_BENCH_UNFUSED_ROPE"))
    ex = g.compiler().compile("cuda", "flat", [])
    gen = torch.Generator(device="cuda")
    gen.manual_seed(rank)
    dt = torch.bfloat16
    for name, shape in weight_inputs(cfg):
        w = torch.empty(shape, dtype=torch.float32, device="cuda").normal_(0.0, 0.02, generator=gen)
        if "norm" in name:
            w += 1.0
        w = w.to(dt)
        ex.set_input_blob(index[name], w.data_ptr(), w.numel() * 2)
        del w
    torch.cuda.empty_cache()
    rng = np.random.default_rng(rank)
    ids = rng.integers(0, cfg.vocab, (B * S,)).astype(np.int64)
    ex.set_input(index["positions"], np.tile(np.arange(S, dtype=np.int64), B))
    ex.set_input(index["last"], (np.arange(B, dtype=np.int64) + 1) * S - 1)
    ex.set_input(index["ids"], ids)
    stream = torch.cuda.ExternalStream(ex.cuda_stream())
    K, W = steps, max(warmup, 3)
    l0 = lib.rg_b200_launch_count()
    ex.run()
    ex.sync()
    launches_per_step = int(lib.rg_b200_launch_count() - l0)
    for _ in range(W):
        ex.run()
    ex.sync()
    sampler = ClockSampler(local)
    sampler.start()

    def block():
        for _ in range(K):
            ex.run()
    ms_blocks, windows = timed_blocks(torch, dist, world, stream, sampler, repeats, lambda: None, block)
    raw = ex.get_output(index["logits"])
    logits_finite = bool(torch.isfinite(torch.from_numpy(raw.view(np.int16)).view(torch.bfloat16).float()).all())
    # end to end: token ids from pinned host memory every step, next tokens read back
    pin_in = torch.from_numpy(ids.copy()).pin_memory()
    pin_out = torch.zeros(B, dtype=torch.int64).pin_memory()
    _barrier(torch, dist, world)
    t0 = time.perf_counter()
    for _ in range(K):
        ex.set_input_async(index["ids"], pin_in.data_ptr(), ids.nbytes)
        ex.run()
        ex.get_output_into(index["next"], pin_out.data_ptr(), B * 8)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1000.0
    clocks, samples = sampler.stop()
    _barrier(torch, dist, world)
    (e2e_ms,) = _max_over_ranks(torch, dist, world, [e2e_ms])
    del ex
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    ms_step, rep = block_summary(ms_blocks, windows, K, samples)
    H, F, V, L, D = cfg.hidden, cfg.ffn, cfg.vocab, cfg.layers, cfg.head_dim
    n = B * S
    gemm_flops = 2.0 * n * L * (3 * H * H + H * H + 3 * H * F) + 2.0 * B * H * V     # LM head on the last token of each sequence
    attn_flops = L * B * cfg.heads * 4.0 * D * (S * (S + 1) / 2.0)
    flops = gemm_flops + attn_flops
    peak, peak_kind = tensor_peak()
    tf = flops / (ms_step * 1e-3) / 1e12
    line = {"metric": "prefill_tokens_per_s", "value": n * world / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": workload_name("7b-prefill"),
                       "logits_finite": logits_finite, "l2": "inputs larger than L2 (13.2 GB of weights, 64 MiB activations per tensor)",
                       "parallelism": "one independent replica per GPU" if world > 1 else "single GPU"},
            "e2e": {"value": K * n * world / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(ids.nbytes), "d2h_bytes_per_step": B * 8},
            "gpu_launches": launches_per_step * K * repeats, "launches_per_step": launches_per_step, "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": None,
                         "kernel": "whole prefill step (gemm_tc_kernel dominates)", "peak_source": peak_kind + " bf16 matmul",
                         "flops_per_step": flops, "gemm_flops": gemm_flops, "attention_flops": attn_flops}}
    line.update(rep)
    return line


def tp_parity_check(torch, dist, lib, comm, rank, world):
    """Outside every timed region: (1) the reference's all-reduce test vector, {2,3} + {5,6} = {7,9}
    (src/04kernel/test/kernels/all_reduce/test_allreduce_nccl.cpp:44-47), continued to `world` ranks (rank r holds
    {2 + 3r, 3 + 3r}); (2) one decode step of a small 2-layer model sharded over the ranks against the oracle's
    tensor-parallel restatement (rank 0 runs it), logits within max-abs 2e-2 / relative 1e-2 and bit-identical on every
    rank.  The oracle is used here as the checker only."""
    from refactorgraph_b200 import capi
    from refactorgraph_b200.llama import LlamaConfig, decode_step_graph_batched, seeded_weights, shard_config, shard_weights, weight_inputs
    out = {}
    x = torch.tensor([2.0 + 3 * rank, 3.0 + 3 * rank], device="cuda")
    y = torch.zeros_like(x)
    comm.all_reduce(capi.F32, 0, 2, x.data_ptr(), y.data_ptr())
    torch.cuda.synchronize()
    want = [sum(2.0 + 3 * r for r in range(world)), sum(3.0 + 3 * r for r in range(world))]
    out["all_reduce_kat"] = y.cpu().tolist() == want
    cfg = LlamaConfig(layers=2, hidden=512, heads=16, kv_heads=8, head_dim=128, ffn=1024, vocab=2000, max_seq=128, batch=16)
    rng = np.random.default_rng(3)
    w16 = seeded_weights(cfg, 0, np.float16)
    w16["lm_head"] = (0.2 * rng.standard_normal(w16["lm_head"].shape)).astype(np.float16)
    B = cfg.batch
    past = rng.integers(1, 100, (B,)).astype(np.int64)
    kc = [rng.standard_normal((B, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    vc = [rng.standard_normal((B, cfg.kv_heads, cfg.max_seq, cfg.head_dim)).astype(np.float16) for _ in range(cfg.layers)]
    token = rng.integers(0, cfg.vocab, (B,)).astype(np.int64)
    sc, kr = shard_config(cfg, world), cfg.kv_heads // world
    ws = shard_weights(cfg, w16, world, rank)
    g, index = decode_step_graph_batched(sc, world=world)
    ex = g.compiler().compile("cuda", "flat", [])
    ex.set_communicator(comm.address)
    for name, _ in weight_inputs(sc):
        ex.set_input(index[name], np.ascontiguousarray(ws[name]))
    for l in range(cfg.layers):
        ex.set_input(index[f"l{l}.k_cache"], np.ascontiguousarray(kc[l][:, rank * kr:(rank + 1) * kr]))
        ex.set_input(index[f"l{l}.v_cache"], np.ascontiguousarray(vc[l][:, rank * kr:(rank + 1) * kr]))
    ex.set_input(index["token"], token)
    ex.set_input(index["pos"], past)
    ex.set_input(index["lens"], past + 1)
    dist.barrier()
    ex.run()
    logits = ex.get_output(index["logits"])
    gathered = [None] * world
    dist.all_gather_object(gathered, logits.tobytes())
    out["bit_identical_across_ranks"] = all(gb == gathered[0] for gb in gathered)
    if rank == 0:
        from oracle.decode_loop import KvHistory, oracle_decode_step_rounded
        r16 = lambda a: np.asarray(a, np.float32).astype(np.float16).astype(np.float32)
        kh = [[KvHistory(kc[l][b], past[b]) for b in range(B)] for l in range(cfg.layers)]
        vh = [[KvHistory(vc[l][b], past[b]) for b in range(B)] for l in range(cfg.layers)]
        wf = {k: v.astype(np.float32) for k, v in w16.items()}
        want_logits = oracle_decode_step_rounded(cfg, wf, kh, vh, token, past, r16, world=world)
        got = logits.astype(np.float32)
        out["max_abs_err_vs_oracle"] = float(np.abs(got - want_logits).max())
        out["decode_step_vs_oracle"] = bool(np.allclose(got, want_logits, atol=2e-2, rtol=1e-2))
    flags = [None] * world
    dist.all_gather_object(flags, out)
    del ex
    merged = dict(flags[0])
    merged["all_reduce_kat"] = all(f["all_reduce_kat"] for f in flags)
    merged["bit_identical_across_ranks"] = all(f["bit_identical_across_ranks"] for f in flags)
    merged["ok"] = bool(merged["all_reduce_kat"] and merged["bit_identical_across_ranks"] and merged.get("decode_step_vs_oracle", False))
    return merged


def time_all_reduce(torch, dist, comm, rank, world, count, launches=50):
    """The all-reduce of the tensor-parallel step alone (fp16, residual add fused), `launches` calls back to back on every
    rank: device microseconds per call, max over ranks."""
    from refactorgraph_b200 import capi
    x = torch.randn(count, device="cuda").to(torch.float16)
    r = torch.randn(count, device="cuda").to(torch.float16)
    y = torch.empty_like(x)
    sid = torch.cuda.current_stream().cuda_stream
    for _ in range(5):
        comm.all_reduce(capi.FP16, 0, count, x.data_ptr(), y.data_ptr(), r.data_ptr(), stream=sid)
    _barrier(torch, dist, world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        comm.all_reduce(capi.FP16, 0, count, x.data_ptr(), y.data_ptr(), r.data_ptr(), stream=sid)
    e1.record()
    torch.cuda.synchronize()
    (us,) = _max_over_ranks(torch, dist, world, [1000.0 * e0.elapsed_time(e1) / launches])
    return us


def measure_decode(args, torch, dist, lib, rank, world, local, workload, steps, warmup, repeats, with_cpu_baseline):
    """One decode workload: device-resident loop (`value`), host-fed loop (`e2e`), the dominant kernel alone (`roofline`).
    `7b` at world > 1 = one independent replica per GPU; `70b-tp` = one model sharded over the ranks."""
    from refactorgraph_b200 import capi
    tp = workload == "70b-tp"
    shard_of = getattr(args, "shard_of", 0) if (tp and world == 1) else 0
    full_cfg, kv_len = workload_config(workload, max(world, shard_of))
    comm, parity, ar_us = None, None, None
    if tp and world > 1:
        def exchange(handle):
            out = [None] * world
            dist.all_gather_object(out, handle)
            return out
        comm = capi.Comm(world, rank, full_cfg.batch * full_cfg.hidden * 2, exchange=exchange)
        parity = tp_parity_check(torch, dist, lib, comm, rank, world)
        ar_us = time_all_reduce(torch, dist, comm, rank, world, full_cfg.batch * full_cfg.hidden)
    ex, index, state = build_executor(full_cfg, kv_len, torch, workload, world, rank, args.graph, shard_of)
    single = workload in ("7b", "tiny", "7b-4l") and args.graph == "single"
    cfg = state["cfg"]                      # per-rank shape
    if comm is not None:
        ex.set_communicator(comm.address)
    stream = torch.cuda.ExternalStream(ex.cuda_stream())
    # tensor-parallel ranks must feed identical tokens; replicas draw their own
    token0 = np.random.default_rng(0 if tp else rank).integers(0, cfg.vocab, (cfg.batch,)).astype(np.int64)
    K, W = steps, max(warmup, 3)
    if int(state["lens0"].max()) + W + K + 8 > cfg.max_seq:
        raise SystemExit("bench.py: steps exceed the KV cache capacity of this benchmark configuration")

    # launches per step, counted on the eager first pass
    reset_state(ex, index, state, token0)
    _barrier(torch, dist, world)
    l0 = lib.rg_b200_launch_count()
    ex.run()
    ex.sync()
    launches_per_step = int(lib.rg_b200_launch_count() - l0)

    # ---- device-resident loop: `repeats` blocks of K steps, every block restarted from the same state ----
    for _ in range(W):
        ex.run()
    ex.sync()
    sampler = ClockSampler(local)
    sampler.start()

    def block():
        for _ in range(K):
            ex.run()
    ms_blocks, windows = timed_blocks(torch, dist, world, stream, sampler, repeats, lambda: reset_state(ex, index, state, token0), block)
    last_tokens = ex.get_output(index["next"]).ravel().tolist()[:8]
    logits_finite = bool(np.isfinite(ex.get_output(index["logits"]).astype(np.float32)).all())
    if not logits_finite:
        raise SystemExit("bench.py: non-finite logits after the timed loop; the number would be meaningless")

    # ---- end-to-end loop: tokens from pinned host memory each step, sampled tokens read back ----
    pin_in = torch.from_numpy(token0.copy()).pin_memory()
    pin_out = torch.zeros(ex.get_output(index["next"]).size, dtype=torch.int64).pin_memory()
    nbytes_in, nbytes_out = cfg.batch * 8, pin_out.numel() * 8

    def e2e_block(n):
        for _ in range(n):
            ex.set_input_async(index["token"], pin_in.data_ptr(), nbytes_in)
            ex.run()
            ex.get_output_into(index["next"], pin_out.data_ptr(), nbytes_out)   # synchronises
            pin_in.copy_(pin_out.view(cfg.batch, -1)[:, 0])
    reset_state(ex, index, state, token0)
    e2e_block(3)
    e2e_ms_blocks = []
    for _ in range(repeats):
        reset_state(ex, index, state, token0)
        pin_in.copy_(torch.from_numpy(token0))
        _barrier(torch, dist, world)
        t0 = time.perf_counter()
        e2e_block(K)
        torch.cuda.synchronize()
        e2e_ms_blocks.append((time.perf_counter() - t0) * 1000.0)
    clocks, samples = sampler.stop()
    _barrier(torch, dist, world)
    e2e_ms_blocks = _max_over_ranks(torch, dist, world, e2e_ms_blocks)
    lin = None
    if rank == 0:
        lin = time_linear_kernel(ex, index, cfg, torch, stream) if workload in ("7b", "tiny", "7b-4l") else time_skinny_gemm(ex, index, cfg, torch, stream)
        att = time_paged_attention(cfg, state["lens0"], torch, stream) if workload == "7b-b32" else None
    comm_ok = comm.status() == capi.OK if comm is not None else True
    err_state = lib.rg_b200_error_state()
    del ex
    torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
    if comm is not None:
        comm.destroy()
    if rank != 0:
        return None

    peak, peak_kind = measured_peak()
    replicas = 1 if tp else world
    ms_step, rep = block_summary(ms_blocks, windows, K, samples)
    value = cfg.batch * replicas / (ms_step * 1e-3)
    e2e_ms_step = statistics.median(e2e_ms_blocks) / K
    kv_sum = float(state["lens0"].sum()) + cfg.batch * (1 + (K - 1) / 2.0)        # mean total cached tokens per step
    step_bytes = cfg.weight_bytes_per_step + cfg.kv_bytes_per_token * kv_sum           # per GPU
    kernel = "linear_stream_kernel" if workload in ("7b", "tiny", "7b-4l") else "gemm_tc_kernel (activations on the N side)"
    roof = {"bound": "hbm", "achieved": lin["gbs"], "peak": peak, "unit": "GB/s", "frac": lin["gbs"] / peak,
            "traffic": None, "kernel": kernel, "peak_source": peak_kind + " HBM copy bandwidth",
            "avg_launch_us": lin["avg_launch_us"], "launches_timed": lin["launches"],
            "algorithmic_bytes_per_launch": lin["bytes_per_pass"] / lin["launches"]}
    if single:
        # the step IS one launch of the dominant kernel: its duration is the CUDA-event time of a timed block / K
        step_gbs = step_bytes / (ms_step * 1e-3) / 1e9
        ratio = ncu_traffic_ratio("decode_mega_7b_4layers_ncu")       # DRAM bytes per algorithmic byte, 4-layer capture; grows with the layer count
        roof = {"bound": "hbm", "achieved": step_gbs, "peak": peak, "unit": "GB/s", "frac": step_gbs / peak,
                "traffic": step_bytes * ratio if ratio else None,
                "kernel": "decode_mega_kernel (one launch per token)", "peak_source": peak_kind + " HBM copy bandwidth",
                "avg_launch_us": 1000.0 * ms_step, "launches_timed": K * repeats, "algorithmic_bytes_per_launch": step_bytes,
                "linear_stream_kernel_alone_gbs": lin["gbs"]}
    elif workload == "7b":
        ratio = ncu_traffic_ratio("linear_gate_up")
        roof["traffic"] = ratio * roof["algorithmic_bytes_per_launch"] if ratio else None
    elif workload == "7b-b32" and att is not None:
        # attention over the paged cache has the largest share of this step (54 % in the ncu launch list); the products come second
        roof = {"bound": "hbm", "achieved": att["gbs"], "peak": peak, "unit": "GB/s", "frac": att["gbs"] / peak, "traffic": None,
                "kernel": "attn_decode_mma_kernel (flash-decoding over the paged cache)", "peak_source": peak_kind + " HBM copy bandwidth",
                "avg_launch_us": att["avg_launch_us"], "launches_timed": att["launches"], "algorithmic_bytes_per_launch": att["bytes_per_launch"],
                "second_kernel": roof}
    line = {
        "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if tp else "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic",
        "config": {"workload": workload_name(workload), "layers": cfg.layers, "hidden": cfg.hidden, "batch": cfg.batch,
                   "logits_finite": logits_finite, "kv_len_start": int(state["lens0"].mean()),
                   "l2": "inputs larger than L2 (all weights streamed once per step)",
                   "parallelism": (f"tp{world}" if tp else ("one independent replica per GPU" if world > 1 else "single GPU")),
                   "last_tokens": last_tokens, "bounded_waits_ok": bool(comm_ok and err_state == 0)},
        "e2e": {"value": cfg.batch * replicas / (e2e_ms_step * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": nbytes_in, "d2h_bytes_per_step": nbytes_out},
        "gpu_launches": launches_per_step * K * repeats,
        "launches_per_step": launches_per_step,
        "clocks": clocks,
        "roofline": roof,
        "roofline_step": {"algorithmic_bytes_per_step_per_gpu": step_bytes, "achieved_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
                          "frac_of_measured": step_bytes / (ms_step * 1e-3) / 1e9 / peak,
                          "frac_of_nominal_8tbs": step_bytes / (ms_step * 1e-3) / 1e9 / 8000.0},
    }
    line.update(rep)
    line["config"]["graph"] = args.graph if workload in ("7b", "tiny", "7b-4l") else "batched"
    if tp:
        line["tp_parity"] = parity
        line["all_reduce_us"] = ar_us
    if shard_of:
        line["diagnostic"] = f"one rank's share of a tp{shard_of} step on one GPU, all-reduce left out: not a benchmark value"
        line["config"]["parallelism"] = f"shard 0 of tp{shard_of}, no exchange"
    if with_cpu_baseline and workload in ("7b", "tiny", "7b-4l"):
        line["cpu_baseline"] = cpu_baseline(cfg, kv_len)
    return line


def _brief(line, keys=("metric", "value", "unit", "ms_per_step", "steps", "warmup", "repeats", "repeat_ms_per_step", "repeat_spread", "repeat_sm_mhz",
                       "dtype", "config", "e2e", "launches_per_step", "clocks", "roofline", "roofline_step", "tp_parity", "all_reduce_us")):
    return {k: line[k] for k in keys if k in line}


def run_b200(args):
    import torch
    import torch.distributed as dist
    from refactorgraph_b200 import capi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernel library has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        # NCCL is only the plumbing here (barriers, max-over-ranks of the timings); IPC handles travel through it too
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = capi.load()
    if args.case == "all_reduce":
        return run_all_reduce_case(args, torch, dist, rank, world)
    R = max(1, args.repeats)
    if args.workload == "7b-prefill":
        line = measure_prefill(args, torch, dist, lib, rank, world, local, args.steps, args.warmup, R)
    else:
        line = measure_decode(args, torch, dist, lib, rank, world, local, args.workload, args.steps, args.warmup, R, not args.no_cpu_baseline)
    # The default run also covers the other configurations, attached to the same JSON line: at one GPU the batch-32 decode,
    # the bf16 prefill and the 10-layer slice of the 70B-shaped model; at N > 1 the 70B-shaped model tensor-parallel over the
    # N GPUs (`value` stays the replica measurement).
    if args.workload == "7b" and not args.only_headline:
        extra = {}
        if world == 1:
            extra["7b-b32"] = measure_decode(args, torch, dist, lib, rank, world, local, "7b-b32", 16, 3, 3, False)
            extra["7b-prefill"] = measure_prefill(args, torch, dist, lib, rank, world, local, 3, 3, 3)
        tpl = measure_decode(args, torch, dist, lib, rank, world, local, "70b-tp", 16, 3, 3, False)
        if rank == 0:
            if extra:
                line["workloads"] = {k: _brief(v) for k, v in extra.items()}
            line["tensor_parallel"] = _brief(tpl)
            line["tensor_parallel"]["tokens_per_s"] = tpl["value"]
            line["gpu_launches"] += sum(v["gpu_launches"] for v in extra.values()) + tpl["gpu_launches"]
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    # Libraries print to descriptor 1 too (NCCL's version banner with NCCL_DEBUG=VERSION): they get stderr, and the JSON line
    # goes to the real stdout through sys.stdout.
    sys.stdout.flush()
    real = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(real, "w", buffering=1)
    if args.case and args.case != "all_reduce":   # all_reduce needs the process group: run_b200 dispatches it
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
