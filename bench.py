#!/usr/bin/env python
"""Benchmark of the decode-time MLA + DSA KV-cache path (one layer-step per "step").

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg3|cfg2|cfg1|cfg4|cfg5|v4]

A layer-step = append one token per sequence -> indexer q quant + score + exact top-k ->
gather/dequant + MLA attention -> bf16 out, over the whole batch. Default workload is the sparse DSA decode
layer the metric is quoted on (batch 128 x context 16384, top-k 2048, 64-token pages scattered over a pool 1.25x
the live set). With N > 1 (one process per GPU under torchrun) the batch of 128 is sharded by sequence over the
ranks - 128 / N sequences each, no collective on the data path: STRONG scaling - and the value is whole-batch
layer-steps/s, timed on the device and reduced with MAX over ranks. The same line then also carries, under
`weak_scaling`, the figure with 128 sequences on every rank, and, under `cfg4`, the long-context case (batch 4 x
context 131,072 sharded by page range, two NCCL all-gathers per step inside the library).

The timed region is R back-to-back repetitions of the K-step loop inside one CUDA-event pair (R sized for at least
0.25 s), so the clock sampler has samples inside it. Before timing, one step at the benchmark's own size is checked
against the oracle on two sampled sequences. Prints ONE JSON line on rank 0. `--workload cfg5` (continuous batching
with churn, one 32-sequence slice per rank) and `--workload v4` (the V4 cousin path) print the same kind of line;
they are not the headline metric.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B per GPU, context after append, heads, index heads, index dim, page, top_k, seed
    "cfg1": dict(B=1, ctx=257, n_heads=16, index_heads=8, index_dim=64, page_tokens=16, top_k=64, seed=0),
    "cfg2": dict(B=32, ctx=2048, n_heads=64, index_heads=32, index_dim=128, page_tokens=64, top_k=2048, seed=1),
    "cfg3": dict(B=128, ctx=16384, n_heads=64, index_heads=32, index_dim=128, page_tokens=64, top_k=2048, seed=2),
    # continuous batching with churn: 78 layers, 32 sequences per GPU (256 over 8 GPUs), ragged contexts U[512, 32768]
    # (pools and tables leave every sequence 64 tokens to grow)
    "cfg5": dict(B=32, ctx_lo=512, ctx_hi=32768, layers=78, n_heads=64, index_heads=32, index_dim=128, page_tokens=64,
                 top_k=2048, seed=4),
    # long context, page-range sharded: every rank holds 1/N of every sequence's pages; candidates and partial
    # attention outputs are exchanged (NCCL all-gather) and merged; needs --gpus >= 2 under torchrun
    "cfg4": dict(B=4, ctx=131072, n_heads=64, index_heads=32, index_dim=128, page_tokens=64, top_k=2048, seed=3),
    # the V4 cousin path (a next-row measurement, not the headline): MQA over one shared 512-wide bf16 entry per
    # position, 128-slot ring + 512 scored compressed blocks of a ratio-4 compressor, 64-head block indexer
    "v4": dict(B=128, ctx=8192, n_heads=64, head_dim=512, window=128, index_heads=64, index_dim=128, index_topk=512,
               ratio=4, seed=5),
}
KV_LORA, ROPE = 512, 64
# dram__bytes_read.sum + dram__bytes_write.sum per launch and per sequence of the cfg3 shape, from ncu captures of
# these kernels at batch 32 (traffic grows in proportion to the sequences a launch processes; a full launch is the
# per-sequence figure x the batch): profiles/ncu_hot_kernels_cfg3_batch32.md
TRAFFIC_PER_SEQ = {"index_score_mma_kernel": (67.31e6 + 0.91e6) / 32, "attend_mma_kernel": (46.23e6 + 0.12e6) / 32,
                   "index_select_cluster_kernel": 4.86e6 / 32}
TRAFFIC_SOURCE = "ncu dram read+write of one launch at batch 32 of the cfg3 shape, per sequence x batch (profiles/ncu_hot_kernels_cfg3_batch32.md)"
METRIC = "DSA decode layer-steps/s (batch×ctx)"


def config_of(name, w, world, B_rank, scaling):
    """The `config` object of the JSON line; both arms print the same one."""
    ctx = w["ctx"]
    total = B_rank * world
    how = (f"batch {total} in total, {B_rank} per GPU (sharded by sequence, no collective)" if scaling == "strong" and world > 1
           else f"batch {B_rank}/GPU")
    return {"workload": f"{name}: {how} x ctx {ctx}, top-k {w['top_k']}, "
                        f"{w['page_tokens']}-token pages scattered in a 1.25x pool, seed {w['seed']}",
            "l2": "inputs larger than L2 (index keys + latents >> 126 MB)" if B_rank * ctx * 132 > 2e8
                  else "working set fits L2: latency-bound config",
            "sequences_per_step": total}


def algorithmic_bytes(w):
    """Per-sequence algorithmic bytes of one layer-step, by stage (append, index, attend)."""
    nt, k, H, nh, hd = w["ctx"], w["top_k"], w["n_heads"], w["index_heads"], w["index_dim"]
    n_sel = min(k, nt)
    W = KV_LORA + ROPE
    append = W * 2 + hd * 2 + 4 + W + 4 + hd + 4
    index = nt * (hd + 4) + nh * hd * 2 + nh * 4 + n_sel * 4
    attend = n_sel * (W + 4) + H * W * 2 + n_sel * 4 + H * KV_LORA * 2
    return dict(append=append, index=index, attend=attend)


def kernel_bytes(w):
    """Per-sequence algorithmic bytes of each KERNEL of the fused step (what it must read and write once)."""
    nt, k, H, nh, hd = w["ctx"], w["top_k"], w["n_heads"], w["index_heads"], w["index_dim"]
    n_sel = min(k, nt)
    W = KV_LORA + ROPE
    return {"step_prologue_kernel": W * 2 + hd * 2 + 4 + W + 4 + hd + 4 + nh * hd * 2 + nh * 4,
            "index_score_mma_kernel": nt * hd + nh * hd,                 # key codes + query codes (scores are not counted)
            "index_select_cluster_kernel": nt * 4 + n_sel * 4,           # key scales + rows out
            "attend_mma_kernel": n_sel * (W + 4) + H * W * 2 + n_sel * 4 + H * KV_LORA * 2}


def algorithmic_flops(w):
    nt, k, H, nh, hd = w["ctx"], w["top_k"], w["n_heads"], w["index_heads"], w["index_dim"]
    n_sel = min(k, nt)
    return dict(index=2 * nh * hd * nt, attend=2 * H * n_sel * (KV_LORA + ROPE + KV_LORA))


KERNELS = ["step_prologue_kernel", "index_score_mma_kernel", "index_select_cluster_kernel", "attend_mma_kernel"]


class ClockSampler:
    """Samples SM clock, power and clock-event reasons of one GPU through NVML (read-only queries)
    from a thread, about every millisecond, so that even a timed region of a few milliseconds
    holds samples; ``mark()`` brackets the timed region. Falls back to ``nvidia-smi -lms``."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.samples, self.marks, self.extra = gpu_index, None, [], [], []
        self.stop_flag, self.h, self.nv, self.t, self.max_mhz = False, None, None, None, None

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            try:
                return int(vis.split(",")[self.idx])
            except (ValueError, IndexError):
                return None          # UUID list: use nvidia-smi's own mapping instead
        return self.idx

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            pi = self._physical_index()
            if pi is None:
                raise RuntimeError("no index")
            self.h, self.nv = nv.nvmlDeviceGetHandleByIndex(pi), nv
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM))
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return
        except Exception:
            self.nv = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _poll(self):
        nv, h = self.nv, self.h
        mask, i = 0, 0
        while not self.stop_flag:
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                if i % 16 == 0:
                    try:
                        self.extra.append((time.perf_counter(), float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_MEM)),
                                           nv.nvmlDeviceGetPowerUsage(h) / 1000.0))
                    except Exception:
                        pass
                if i % 4 == 0:          # the reasons query is the slower of the two
                    try:
                        mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                    except Exception:
                        mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                self.samples.append((time.perf_counter(), mhz, mask))
            except Exception:
                pass
            i += 1
            time.sleep(0.0002)

    def _read(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        bits = {v: k for k, v in self.REASONS.items()}
        for ln in self.proc.stdout:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                mhz, mx = float(f[1]), float(f[2])
            except ValueError:
                continue
            self.max_mhz = max(self.max_mhz or 0.0, mx)
            mask = sum(bits[n] for n, v in zip(names, f[5:9]) if v.lower().startswith("active"))
            self.samples.append((time.perf_counter(), mhz, mask))

    def mark(self):
        self.marks.append(time.perf_counter())

    def stop(self):
        self.stop_flag = True
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        if self.t:
            self.t.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        lo, hi = (self.marks + [None, None])[:2]
        inside = [s for s in self.samples if lo is not None and hi is not None and lo <= s[0] <= hi]
        use = inside or self.samples          # a region shorter than the sampling period: the whole loaded phase
        mask = 0
        for s in use:
            mask |= s[2]
        out = {"sm_mhz": float(np.median([s[1] for s in use])), "sm_max_mhz": self.max_mhz,
               "reasons": sorted(n for b, n in self.REASONS.items() if mask & b),
               "samples": len(use), "samples_in_timed_region": len(inside),
               "source": "nvml" if self.nv else "nvidia-smi"}
        ex = [e for e in self.extra if lo is not None and hi is not None and lo <= e[0] <= hi]
        if ex:
            out["mem_mhz"] = float(np.median([e[1] for e in ex]))
            out["power_w_max"] = float(max(e[2] for e in ex))
        return out


def build_layer(w, device, seed):
    """Device state for one workload: pools filled on the GPU by the append kernel."""
    import torch
    from rivoli_b200 import backend as be
    from rivoli_b200.layer import DsaDecodeLayer

    B, ctx, P = w["B"], w["ctx"], w["page_tokens"]
    pages_per_seq = (ctx + P - 1) // P
    live = B * pages_per_seq
    n_pool = max(int(np.ceil(live * 1.25)), live)
    g = be.DsaGeom.make(n_heads=w["n_heads"], kv_lora=KV_LORA, rope_dim=ROPE, index_heads=w["index_heads"],
                        index_dim=w["index_dim"], page_tokens=P, top_k=w["top_k"],
                        max_pages_per_seq=pages_per_seq, n_pool_pages=n_pool)
    layer = DsaDecodeLayer(g, B, device=device, max_ctx=ctx, shuffle_seed=seed * 7919 + 17)
    for b in range(B):
        layer.reserve(b, ctx)
    layer.upload_block_table()
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    W = KV_LORA + ROPE
    # history: ctx-1 tokens per sequence, appended in chunks to bound scratch memory
    chunk = 1 << 16
    total = B * (ctx - 1)
    for s0 in range(0, total, chunk):
        n = min(chunk, total - s0)
        idx = torch.arange(s0, s0 + n, device=device, dtype=torch.int64)
        seq = (idx // (ctx - 1)).to(torch.int32)
        pos = (idx % (ctx - 1)).to(torch.int32)
        lat = torch.randn((n, W), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
        key = torch.randn((n, w["index_dim"]), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
        layer.append(lat, key, pos, seq)
    torch.cuda.synchronize(device)
    layer.check_status()
    return g, layer, gen


def step_inputs(w, device, gen, pinned=False):
    import torch
    B, W = w["B"], KV_LORA + ROPE
    mk = lambda *s: torch.randn(s, generator=gen, device=device, dtype=torch.float32)
    d = dict(latent=mk(B, W).to(torch.bfloat16), index_key=mk(B, w["index_dim"]).to(torch.bfloat16),
             index_q=mk(B, w["index_heads"], w["index_dim"]).to(torch.bfloat16),
             index_w=mk(B, w["index_heads"]).to(torch.bfloat16).to(torch.float32),
             q=mk(B, w["n_heads"], W).to(torch.bfloat16))
    if pinned:
        return {k: v.cpu().pin_memory() for k, v in d.items()}
    return d


def self_check(layer, g, w, x, row_pos, seq_len, seqs):
    """Parity of ONE step at the benchmark's own size, outside any timed region: for the sampled sequences the
    oracle runs the same step on a copy of their pages (append, scores, exact top-k, attention) and the GPU's
    appended codes and scales, selected rows (bit for bit) and attention output (2e-2 relative / 1e-3 absolute,
    elementwise) must agree. The pages are copied BEFORE the step; the step itself is the timed call."""
    import torch
    from oracle import oracle as orc
    from oracle.workload import attend_close, make_geom
    P, W, hd = g.page_tokens, KV_LORA + ROPE, g.index_dim
    n_pages = (int(seq_len.max().item()) + P - 1) // P
    seqs = list(seqs)
    pages = layer.block_table[seqs, :n_pages].long().reshape(-1)                   # device
    take = lambda pool, width: pool.view(g.n_pool_pages, P * width)[pages].cpu().numpy().reshape(-1)
    lp, ls = take(layer.latent_pool, W), layer.latent_scale.view(g.n_pool_pages, P)[pages].cpu().numpy().reshape(-1)
    ip, isc = take(layer.index_pool, hd), layer.index_scale.view(g.n_pool_pages, P)[pages].cpu().numpy().reshape(-1)
    n = len(seqs)
    bt = np.arange(n * n_pages, dtype=np.int32).reshape(n, n_pages)
    og = make_geom(orc.Geom, n_heads=g.n_heads, index_heads=g.index_heads, index_dim=hd, page_tokens=P, top_k=g.top_k,
                   max_pages_per_seq=n_pages, n_pool_pages=n * n_pages)
    u16 = lambda t: t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
    rp, sl = row_pos[seqs].cpu().numpy(), seq_len[seqs].cpu().numpy()
    assert orc.kv_append_paged(og, u16(x["latent"][seqs]), u16(x["index_key"][seqs]), None, rp, bt, lp, ls, ip, isc) == 0
    qc, qs = orc.index_q_quant(u16(x["index_q"][seqs]), hd)
    sc = orc.index_score_paged(og, qc, qs, x["index_w"][seqs].cpu().numpy(), ip, isc, bt, sl, int(sl.max()))
    rows, n_sel = orc.index_topk_batched(sc, sl, g.top_k)
    _, want, _, _ = orc.mla_attend_paged(og, u16(x["q"][seqs]), lp, ls, bt, rows, n_sel, want_f32=True)
    out = layer.step(x["latent"], x["index_key"], x["index_q"], x["index_w"], x["q"], row_pos, seq_len)
    torch.cuda.synchronize(layer.dev)
    layer.check_status()
    assert np.array_equal(take(layer.latent_pool, W), lp), "appended latent codes differ from the oracle"
    assert np.array_equal(layer.latent_scale.view(g.n_pool_pages, P)[pages].cpu().numpy().reshape(-1).view(np.uint32), ls.view(np.uint32))
    assert np.array_equal(take(layer.index_pool, hd), ip), "appended index codes differ from the oracle"
    got_rows = layer.rows[seqs].cpu().numpy().view(np.uint32)
    for i in range(n):
        assert int(layer.n_sel[seqs[i]].item()) == int(n_sel[i])
        assert np.array_equal(got_rows[i, :n_sel[i]], rows[i, :n_sel[i]]), "selected rows differ from the oracle"
    ok, worst = attend_close(u16(out[seqs]), want)
    assert ok, f"attention outside 2e-2 rel / 1e-3 abs (worst err/tol {worst:.2f})"
    return {"sequences": seqs, "codes_scales_rows": "bit-exact", "attention_worst_err_over_tol": round(worst, 3)}


def timed_steps(step, K, R, barrier, device):
    """R back-to-back repetitions of the K-step loop inside ONE event pair (the timed region is then long enough
    for the clock sampler to see it); returns milliseconds per step over all R * K steps."""
    import torch
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(R):
        for _ in range(K):
            step()
    t1.record()
    barrier()
    return t0.elapsed_time(t1) / (R * K)


def kernel_times(layer, step, n, device):
    """Average duration of each kernel of the fused step over n steps, from CUDA events the library records between
    its launches (rivoli_dsa_step_set_timing_events) on the launching stream. Outside the `value` region: the records
    serialise the kernels, which `value` keeps overlapped."""
    import torch
    from rivoli_b200 import backend as be
    sets = []
    for _ in range(n):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        for e in ev:
            e.record()                     # creates the handles
        sets.append(ev)
    torch.cuda.synchronize(device)
    for ev in sets:
        be.step_set_timing_events(ev)
        step()
    be.step_set_timing_events(None)
    torch.cuda.synchronize(device)
    return {k: float(np.mean([ev[i].elapsed_time(ev[i + 1]) for ev in sets])) for i, k in enumerate(KERNELS)}


def measure_layer(w, B, device, seed, args, barrier, sampler=None, check=False, e2e=True):
    """Builds the workload with B sequences on this GPU and measures: device-resident ms/step (fused call), per-kernel
    times, end-to-end ms/step through the host-buffer pipeline."""
    import torch
    from rivoli_b200.layer import HostStepPipeline
    wB = dict(w, B=B)
    g, layer, gen = build_layer(wB, device, seed)
    ctx = w["ctx"]
    x = step_inputs(wB, device, gen)
    row_pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=device)
    seq_len = torch.full((B,), ctx, dtype=torch.int32, device=device)
    res = {"B": B}
    if check:
        res["self_check"] = self_check(layer, g, wB, x, row_pos, seq_len, sorted({0, B - 1}))

    def step():
        # the call a device-resident caller makes: ONE library call, 4 launches (append + query prologue, scorer,
        # selection, tensor-core attention; the short-context attention arm is not launched: the scheduler's
        # lower bound on the context says no sequence needs it)
        layer.step(x["latent"], x["index_key"], x["index_q"], x["index_w"], x["q"], row_pos, seq_len, min_rows_hint=hint)

    hint = min(w["top_k"], ctx)            # what a scheduler knows: every sequence of this batch attends that many rows
    W_ = max(args.warmup, 3)
    for _ in range(W_):
        step()
    barrier()
    layer.check_status()
    # size the repetitions so that the timed region is at least 0.25 s
    t_est = timed_steps(step, 10, 1, barrier, device)
    R = args.reps or max(1, int(np.ceil(250.0 / max(t_est * args.steps, 1e-3))))
    if sampler:
        sampler.start()
        time.sleep(0.05)
        sampler.mark()
    res["ms"] = timed_steps(step, args.steps, R, barrier, device)
    if sampler:
        sampler.mark()
    res["reps"] = R
    res["kernel_ms"] = kernel_times(layer, step, min(args.steps, 50), device)
    barrier()
    layer.check_status()
    if e2e:
        # end to end through the host-facing call: one packed pinned input buffer up, the bf16 output down, every step
        xh = step_inputs(wB, device, gen, pinned=True)
        pipe = HostStepPipeline(layer, depth=2, min_rows_hint=hint)
        packed = [pipe.pack(xh), pipe.pack(xh)]
        outs_h = [pipe.new_output_buffer() for _ in range(2)]
        torch.cuda.synchronize(device)
        i_ = [0]

        def e2e_step():
            pipe.submit(packed[i_[0] & 1], outs_h[i_[0] & 1], row_pos, seq_len)
            i_[0] += 1

        for _ in range(4):
            e2e_step()
        pipe.drain()
        barrier()
        n_e2e = args.steps * max(1, R // 4)
        t0 = time.perf_counter()          # host clock around a fully drained pipeline: submit never blocks, drain does
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        s_up = torch.cuda.ExternalStream(pipe.pipe.stream(0), device=device)
        s_down = torch.cuda.ExternalStream(pipe.pipe.stream(2), device=device)
        e0.record(s_up)
        for _ in range(n_e2e):
            e2e_step()
        e1.record(s_down)                 # after the last download: every earlier leg precedes it
        pipe.drain()
        res["e2e_wall_ms"] = (time.perf_counter() - t0) * 1e3 / n_e2e
        res["e2e_ms"] = e0.elapsed_time(e1) / n_e2e
        res["e2e_legs_ms"] = pipe.leg_ms()
        res["h2d"] = pipe.pipe.input_bytes
        res["d2h"] = pipe.pipe.output_bytes
        barrier()
        layer.check_status()
        del pipe
    del layer
    torch.cuda.empty_cache()
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist
    from rivoli_b200 import backend as be

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    be.lib()
    w = WORKLOADS[args.workload]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def max_over_ranks(vals):
        if world == 1:
            return [float(v) for v in vals]
        t = torch.tensor(vals, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    sampler = ClockSampler(local) if rank == 0 else None
    # The configuration the metric is quoted on: the workload's batch IN TOTAL, sharded by sequence over the ranks
    # (strong scaling; at N = 1 that is the whole batch on one GPU). Sequences that do not divide evenly go to the
    # lower ranks.
    base, rem = divmod(w["B"], world)
    B_rank = base + (1 if rank < rem else 0)
    strong = measure_layer(w, max(B_rank, 1), device, w["seed"] + 1000 * rank, args, barrier, sampler, check=(rank == 0))
    clocks = sampler.stop() if sampler else None
    ms, ms_e2e, ms_e2e_wall = max_over_ranks([strong["ms"], strong["e2e_ms"], strong["e2e_wall_ms"]])
    weak = None
    if world > 1:
        # secondary figure: the same per-GPU batch on every rank (weak scaling, N independent replicas)
        wk = measure_layer(w, w["B"], device, w["seed"] + 1000 * rank, args, barrier, None, check=False, e2e=False)
        weak_ms, = max_over_ranks([wk["ms"]])
        weak = {"scaling": "weak", "value": world * 1e3 / weak_ms, "unit": "layer-steps/s", "ms_per_step": weak_ms,
                "sequences_per_step": w["B"] * world,
                "what": f"every rank runs the whole batch of {w['B']} on its own sequences (independent replicas)"}
    cfg4 = None
    if world > 1 and args.workload == "cfg3":
        cfg4 = measure_cfg4(args, rank, world, device, steps=min(args.steps, 100), warmup=max(args.warmup, 3))

    if rank == 0:
        ab, af, kb = algorithmic_bytes(w), algorithmic_flops(w), kernel_bytes(w)
        peaks = {}
        pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(pk):
            peaks = json.load(open(pk))
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
        B0 = strong["B"]
        km = strong["kernel_ms"]
        per_kernel = {k: {"us": km[k] * 1e3, "bytes": kb[k] * B0, "gbs": kb[k] * B0 / (km[k] * 1e-3) / 1e9,
                          "frac": kb[k] * B0 / (km[k] * 1e-3) / 1e9 / hbm_peak} for k in KERNELS}
        dom = max(KERNELS, key=lambda k: km[k])                    # the single longest kernel of the step
        value = 1e3 / ms                                           # whole-job layer-steps/s (a layer-step = the whole batch)
        step_bytes = sum(ab.values()) * B0
        line = {
            "metric": METRIC, "value": value, "unit": "layer-steps/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "fp8-e4m3 cache, bf16 activations, f32 accumulate", "data": "synthetic",
            "config": dict(config_of(args.workload, w, world, base if world > 1 else w["B"], "strong"),
                           timed_region=f"{strong['reps']} back-to-back repetitions of the {args.steps}-step loop inside one "
                                        f"CUDA-event pair; ms_per_step is over all of them"),
            "timed_repetitions": strong["reps"],
            "e2e": {"value": 1e3 / ms_e2e, "unit": "layer-steps/s", "h2d_bytes_per_step": strong["h2d"] * (1 if world == 1 else 1),
                    "d2h_bytes_per_step": strong["d2h"], "bytes_are": "per GPU", "ms_per_step": ms_e2e,
                    "ms_per_step_host_clock": ms_e2e_wall, "legs_ms_rank0": strong["e2e_legs_ms"],
                    "call": "rivoli_dsa_step_host: one packed pinned buffer up, fused step, bf16 output down, 3 streams x 2 slots"},
            "gpu_launches": args.steps * strong["reps"] * (4 if min(w["top_k"], w["ctx"]) >= 128 else 5),   # prologue, scorer, selection, (short-context attention arm,) tensor-core attention
            "kernel_us": {k: km[k] * 1e3 for k in KERNELS},
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": per_kernel[dom]["gbs"], "peak": hbm_peak, "unit": "GB/s",
                         "frac": per_kernel[dom]["frac"], "peak_source": f"of {peak_src}",
                         "traffic": TRAFFIC_PER_SEQ.get(dom, 0) * B0 or None,
                         "traffic_source": TRAFFIC_SOURCE,
                         "kernels": per_kernel,
                         "layer_step_bytes": step_bytes,
                         "layer_step_gbs_per_gpu": step_bytes / (ms * 1e-3) / 1e9,
                         "layer_step_frac": step_bytes / (ms * 1e-3) / 1e9 / hbm_peak,
                         "attend_tflops": af["attend"] * B0 / (km["attend_mma_kernel"] * 1e-3) / 1e12},
            "self_check": strong.get("self_check"),
            "clocks": clocks,
        }
        if weak:
            line["weak_scaling"] = weak
        if cfg4:
            line["cfg4"] = cfg4
        if world == 1:
            proj = time_projections(w, device)
            if proj:
                line["next_rows"] = {"what": "q absorption, value up-projection (kv_b) and the indexer front end (two launches), tcgen05 kind::f16, per call "
                                             "at this batch, L2 flushed between launches; not part of the layer-step metric",
                                     **proj}
            if not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_baseline(w, seconds=12.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def time_projections(w, device, steps=50):
    """The rows either side of the cache path (q absorption, value up-projection) at the workload's
    batch: CUDA-event time per launch and algorithmic GB/s. Not part of the layer-step metric."""
    import torch
    from rivoli_b200 import backend as be
    if w["n_heads"] != 64:
        return None
    H, qh, nope, vh, kvl, rope, block, B = 64, 256, 192, 256, KV_LORA, ROPE, 128, w["B"]
    gen = torch.Generator(device=device)
    gen.manual_seed(w["seed"] + 77)
    rows = H * (nope + vh)
    kvb = torch.randint(0, 0x7E, (rows * kvl,), generator=gen, device=device, dtype=torch.int32).to(torch.uint8)
    scale = torch.rand(((rows // block) * (kvl // block),), generator=gen, device=device) * 0.01 + 0.002
    q = torch.randn((B, H, qh), generator=gen, device=device).to(torch.bfloat16)
    clat = torch.randn((B, H, kvl), generator=gen, device=device).to(torch.bfloat16)
    q_abs = torch.empty((B, H, kvl + rope), dtype=torch.bfloat16, device=device)
    ctx = torch.empty((B, H, vh), dtype=torch.bfloat16, device=device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)      # > L2: weights come from HBM each time
    out = {}
    for name, fn, nbytes, flops in (
            ("absorb", lambda: be.launch_mla_absorb_batched_bf16(q, kvb, scale, H, qh, nope, vh, kvl, rope, block, B, q_abs),
             H * nope * kvl + B * H * (nope + rope) * 2 + B * H * (kvl + rope) * 2, 2 * B * H * nope * kvl),
            ("value", lambda: be.launch_mla_value_batched_bf16(clat, kvb, scale, H, nope, vh, kvl, block, B, ctx),
             H * vh * kvl + B * H * kvl * 2 + B * H * vh * 2, 2 * B * H * vh * kvl)):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize(device)
            ts.append(e0.elapsed_time(e1))
        ms = float(np.median(ts))
        out[name] = {"us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9, "tflops": flops / (ms * 1e-3) / 1e12}
    be.kvb_proj_status()
    # indexer front end at the model geometry (hidden 6144, q_lora 2048, 32 x 128 index heads)
    from rivoli_b200.layer import IndexerFrontEnd
    hidden, q_lora, nh, hd = 6144, 2048, w["index_heads"], w["index_dim"]
    fg = be.IndexFrontGeom(hidden, q_lora, nh, hd, 0, 64, block, 1e-6, 10000.0)

    def fp8w(n, k):
        return (torch.randint(0, 0x7E, (n * k,), generator=gen, device=device, dtype=torch.int32).to(torch.uint8),
                torch.rand((((n + block - 1) // block) * (k // block),), generator=gen, device=device) * 0.01 + 0.002)
    wk, wk_s = fp8w(hd, hidden); wq, wq_s = fp8w(nh * hd, q_lora); wp, wp_s = fp8w(nh, hidden)
    fe = IndexerFrontEnd(fg, B, dict(wk=wk, wk_scale=wk_s, knorm_w=torch.ones(hd, device=device), knorm_b=torch.zeros(hd, device=device),
                                     wq_b=wq, wq_b_scale=wq_s, wproj=wp, wproj_scale=wp_s), device=device)
    xh = torch.randn((B, hidden), generator=gen, device=device).to(torch.bfloat16)
    qr = torch.randn((B, q_lora), generator=gen, device=device).to(torch.bfloat16)
    pos = torch.full((B,), w["ctx"] - 1, dtype=torch.int32, device=device)
    nbytes = hd * hidden + nh * hd * q_lora + nh * hidden + B * (hidden + q_lora) * 2 + B * (hd + nh * hd) * 2 + B * nh * 4
    for _ in range(3):
        fe.run(xh, qr, pos)
    ts = []
    for _ in range(steps):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fe.run(xh, qr, pos); e1.record()
        torch.cuda.synchronize(device)
        ts.append(e0.elapsed_time(e1))
    ms = float(np.median(ts))
    be.index_frontend_status()
    out["index_front_end"] = {"us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9,
                              "tflops": 2 * B * (hd * hidden + nh * hd * q_lora + nh * hidden) / (ms * 1e-3) / 1e12}
    return out


def churn_parity_check(device):
    """Continuous batching at reduced scale against the oracle, outside any timed region: 2 layers, 8 slots, contexts
    U[300, 1500], three token-steps with 25 % of the slots replaced after each. Page tables and free list must equal
    the oracle allocator's bit for bit, the selected rows of every layer the oracle's, the attention output within
    2e-2 relative / 1e-3 absolute."""
    import torch
    from oracle import oracle as orc
    from oracle.workload import attend_close, bf16_normal, make_geom
    from rivoli_b200 import backend as be
    from rivoli_b200.engine import DsaDecodeStack
    from rivoli_b200.scheduler import ContinuousBatcher, churn_plan
    n_slots, n_layers, P, top_k, steps, lo, hi = 8, 2, 64, 256, 3, 300, 1500
    max_ctx = hi + steps + 1
    max_pages = (max_ctx + P - 1) // P
    n_pool = int(1.25 * n_slots * max_pages)
    kw = dict(n_heads=64, index_heads=32, index_dim=128, page_tokens=P, top_k=top_k, max_pages_per_seq=max_pages, n_pool_pages=n_pool)
    g, og = make_geom(be.DsaGeom, **kw), make_geom(orc.Geom, **kw)
    stack = DsaDecodeStack(g, n_slots, [True] * n_layers, device=device, max_ctx=max_pages * P, shuffle_seed=4)
    sched = ContinuousBatcher(n_slots, n_pool, max_ctx, P, pool=stack.pool)
    opool = orc.Pool(n_pool, n_slots, max_pages, P)
    opool.shuffle(4)

    class _O:                               # the oracle's allocator behind the scheduler's pool interface
        def reserve(self, s_, n): return opool.reserve(s_, n)
        def release(self, s_): return opool.release(s_)
        def block_table(self): return opool.block_table()
        n_free = property(lambda self: opool.n_free)
    osched = ContinuousBatcher(n_slots, n_pool, max_ctx, P, pool=_O())
    rng = np.random.RandomState(4)
    W, hd = KV_LORA + ROPE, 128
    rows_n = n_pool * P
    mirror = [dict(lp=np.zeros(rows_n * W, np.uint8), ls=np.zeros(rows_n, np.float32), ip=np.zeros(rows_n * hd, np.uint8),
                   isc=np.zeros(rows_n, np.float32)) for _ in range(n_layers)]

    def dev(a):
        a = np.ascontiguousarray(a)
        return torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).to(device)

    def prefill(slots, lens):
        stack.upload_block_table()
        bt = sched.block_table()
        for s_, n in zip(slots, lens):
            pos, seq = np.arange(int(n), dtype=np.int32), np.full(int(n), int(s_), np.int32)
            for L, M in zip(stack.layers, mirror):
                lat, key = bf16_normal(rng, (int(n), W)), bf16_normal(rng, (int(n), hd))
                L.append(dev(lat), dev(key), dev(pos), dev(seq))
                assert orc.kv_append_paged(og, lat, key, seq, pos, bt, M["lp"], M["ls"], M["ip"], M["isc"]) == 0

    first = rng.randint(lo, hi + 1, n_slots)
    for s_, n in enumerate(first):
        sched.admit(s_, int(n)); osched.admit(s_, int(n))
    prefill(range(n_slots), first)
    worst_all = 0.0
    for step in range(steps):
        row_pos, seq_len = sched.begin_step()
        osched.begin_step()
        bt = sched.block_table()
        assert np.array_equal(bt, osched.block_table()), "page tables differ from the oracle allocator"
        assert np.array_equal(stack.pool.free_list(), opool.free_list()), "free lists differ from the oracle allocator"
        stack.upload_block_table()
        for li, (L, M) in enumerate(zip(stack.layers, mirror)):
            lat, key = bf16_normal(rng, (n_slots, W)), bf16_normal(rng, (n_slots, hd))
            iq, iw = bf16_normal(rng, (n_slots, 32, hd)), orc.bf16_to_f32(bf16_normal(rng, (n_slots, 32)))
            q = bf16_normal(rng, (n_slots, 64, W))
            out = stack.step_layer(li, dev(lat), dev(key), dev(iq), dev(iw), dev(q), dev(row_pos), dev(seq_len))
            torch.cuda.synchronize(device)
            L.check_status()
            assert orc.kv_append_paged(og, lat, key, None, row_pos, bt, M["lp"], M["ls"], M["ip"], M["isc"]) == 0
            qc, qs = orc.index_q_quant(iq, hd)
            sc = orc.index_score_paged(og, qc, qs, iw, M["ip"], M["isc"], bt, seq_len, int(seq_len.max()))
            rows, n_sel = orc.index_topk_batched(sc, seq_len, top_k)
            _, want, _, _ = orc.mla_attend_paged(og, q, M["lp"], M["ls"], bt, rows, n_sel, want_f32=True)
            got = L.rows.cpu().numpy().view(np.uint32)
            for b in range(n_slots):
                assert np.array_equal(got[b, :n_sel[b]], rows[b, :n_sel[b]]), "selected rows differ from the oracle"
            ok, worst = attend_close(out.cpu().view(torch.int16).numpy().view(np.uint16), want)
            assert ok, worst
            worst_all = max(worst_all, worst)
        slots, lens = churn_plan(rng, n_slots, 0.25, lo, hi)
        sched.finish(slots, lens); osched.finish(slots, lens)
        prefill(slots, lens)
    del stack
    torch.cuda.empty_cache()
    return {"what": f"{n_layers} layers x {n_slots} slots x {steps} token-steps with 25 % replacement: page tables, free list and "
                    "selected rows bit-exact against the oracle, attention within 2e-2 / 1e-3",
            "attention_worst_err_over_tol": round(worst_all, 3)}


def run_churn(args):
    """Continuous batching with eviction churn: `layers` decode layers behind one page allocator, a ragged
    batch (contexts U[512, 32768]), every token-step appends one token per sequence per layer, selects and
    attends; after each token-step 10 % of the sequences finish, their pages return to the free list and
    replacements with fresh contexts are admitted (their prefill is NOT timed). Under torchrun every rank runs its own
    32-sequence slice of the batch of 256 with its own allocator (sharded by sequence, no collective); the time is the
    MAX over ranks. Prints one JSON line on rank 0."""
    import torch
    import torch.distributed as dist
    from rivoli_b200 import backend as be
    from rivoli_b200.engine import DsaDecodeStack
    from rivoli_b200.scheduler import ContinuousBatcher, churn_plan
    w = WORKLOADS["cfg5"]
    n_layers = args.layers or w["layers"]
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    parity = churn_parity_check(device) if rank == 0 else None
    B, P, lo, hi = w["B"], w["page_tokens"], w["ctx_lo"], w["ctx_hi"]
    max_ctx = 32768 + 64
    assert hi + args.steps + args.warmup < max_ctx, "too many token-steps for the context bound"
    max_pages = (max_ctx + P - 1) // P
    n_pool = int(1.25 * B * max_pages)
    g = be.DsaGeom.make(n_heads=w["n_heads"], kv_lora=KV_LORA, rope_dim=ROPE, index_heads=w["index_heads"],
                        index_dim=w["index_dim"], page_tokens=P, top_k=w["top_k"], max_pages_per_seq=max_pages,
                        n_pool_pages=n_pool)
    seed = w["seed"] + 1000 * rank                 # every rank: its own requests
    stack = DsaDecodeStack(g, B, [True] * n_layers, device=device, max_ctx=max_pages * P, shuffle_seed=seed)
    sched = ContinuousBatcher(B, n_pool, max_ctx, P, pool=stack.pool)
    rng = np.random.RandomState(seed)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    W = KV_LORA + ROPE
    blk = 1 << 15                                  # one block of random rows serves every prefill (contents are irrelevant here)
    lat_blk = torch.randn((blk, W), generator=gen, device=device).to(torch.bfloat16)
    key_blk = torch.randn((blk, w["index_dim"]), generator=gen, device=device).to(torch.bfloat16)

    def prefill(slots, lens):
        stack.upload_block_table()
        for s_, n in zip(slots, lens):
            for o in range(0, int(n), blk):
                m = min(blk, int(n) - o)
                pos = torch.arange(o, o + m, dtype=torch.int32, device=device)
                seq = torch.full((m,), int(s_), dtype=torch.int32, device=device)
                for L in stack.layers:
                    L.append(lat_blk[:m], key_blk[:m], pos, seq)

    first = rng.randint(lo, hi + 1, B)
    for s_, n in enumerate(first):
        sched.admit(s_, int(n))
    prefill(range(B), first)
    x = step_inputs(dict(w, B=B), device, gen)
    torch.cuda.synchronize(device)
    times, appended = [], 0
    for it in range(args.warmup + args.steps):
        row_pos, seq_len = sched.begin_step()          # host: one page-table update for all layers
        rp, sl = torch.from_numpy(row_pos).to(device), torch.from_numpy(seq_len).to(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        stack.upload_block_table()
        for i in range(n_layers):
            stack.step_layer(i, x["latent"], x["index_key"], x["index_q"], x["index_w"], x["q"], rp, sl,
                             min_rows_hint=min(w["top_k"], lo))     # the scheduler's bound: no context below `lo`
        e1.record()
        torch.cuda.synchronize(device)
        if it >= args.warmup:
            times.append(e0.elapsed_time(e1))
            appended += B
        slots, lens = churn_plan(rng, B, 0.10, lo, hi)
        sched.finish(slots, lens)
        prefill(slots, lens)                          # untimed
        torch.cuda.synchronize(device)
    for L in stack.layers[:2]:
        L.check_status()
    ms = float(np.mean(times))
    mean_ctx = float(sched.seq_len.mean())
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        line = {"metric": METRIC, "value": n_layers / (ms * 1e-3), "unit": "layer-steps/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / n_layers, "higher_is_better": True,
                "scaling": "strong" if world > 1 else "weak",
                "vs_baseline": None, "dtype": "fp8-e4m3 cache, bf16 activations, f32 accumulate", "data": "synthetic",
                "config": {"workload": f"cfg5: {n_layers} layers x batch {B * world} ({B}/GPU, sharded by sequence), contexts "
                                       f"U[{lo},{hi}], top-k {w['top_k']}, {P}-token pages from one shared free list per GPU, "
                                       f"10 % of sequences replaced per token-step (prefill untimed), seed {w['seed']}",
                           "token_step_ms": ms, "token_steps_per_s": 1e3 / ms, "tokens_per_s": B * world * 1e3 / ms,
                           "mean_context_rank0": mean_ctx,
                           "a_layer_step_is": f"one layer over the whole batch of {B * world} sequences"},
                "parity": parity,
                "gpu_launches": args.steps * n_layers * 5}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_v4(args):
    """One decode step of the V4 cousin path per "step": block scores + exact top-k selection rows, then sparse
    MQA attention with the sink, for every sequence of the batch. Prints one JSON line (same keys as the
    headline line; the CPU arm is the oracle on a bounded sample of the same sequences)."""
    import torch
    from oracle import oracle as orc
    from oracle import v4_workload as wl
    from rivoli_b200 import backend as be
    from rivoli_b200.v4 import V4DecodeLayer
    w = WORKLOADS["v4"]
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    B, max_comp = w["B"], w["ctx"] // w["ratio"]
    og = wl.make_geom(n_heads=w["n_heads"], head_dim=w["head_dim"], window=w["window"], index_heads=w["index_heads"],
                      index_dim=w["index_dim"], index_topk=w["index_topk"], ratio=w["ratio"], max_comp=max_comp)
    g = be.V4Geom(*[getattr(og, n) for n, _ in orc.V4Geom._fields_])
    pos = np.full(B, w["ctx"] - 1, np.int32)
    n_cpu = 2                                             # sequences the CPU arm and the parity check cover
    host = wl.make_inputs(og, n_cpu, pos[:n_cpu], seed=w["seed"])
    layer = V4DecodeLayer(g, B, device)
    gen = torch.Generator(device=device)
    gen.manual_seed(w["seed"])
    rnd = lambda *shape: torch.randn(shape, generator=gen, device=device).to(torch.bfloat16).view(torch.uint16)
    layer.kv_cache.copy_(rnd(B, layer.kv_rows, g.head_dim))
    spread = torch.randn((B * max_comp, g.index_dim), generator=gen, device=device).to(torch.bfloat16).float()
    be.launch_act_quant_f4_rotated(spread, B * max_comp, g.index_dim)
    layer.index_kv.copy_(spread.to(torch.bfloat16).view(torch.uint16).view(B, max_comp, g.index_dim))
    iq = torch.randn((B * g.index_heads, g.index_dim), generator=gen, device=device).to(torch.bfloat16).float()
    be.launch_act_quant_f4_rotated(iq, B * g.index_heads, g.index_dim)
    iq = iq.to(torch.bfloat16).view(torch.uint16).view(B, g.index_heads, g.index_dim).contiguous()
    iw = (torch.randn((B, g.index_heads), generator=gen, device=device) * g.index_heads ** -0.5).to(torch.bfloat16).float()
    q = rnd(B, g.n_heads, g.head_dim)
    layer.sink.copy_(torch.randn(g.n_heads, generator=gen, device=device))
    # the first n_cpu sequences carry the oracle's inputs so the run checks itself
    for name, dst in (("kv_cache", layer.kv_cache), ("ikv", layer.index_kv), ("iq", iq), ("q", q)):
        dst[:n_cpu].copy_(torch.from_numpy(host[name]).to(device))
    iw[:n_cpu].copy_(torch.from_numpy(host["iw"]).to(device))
    layer.sink.copy_(torch.from_numpy(host["sink"]).to(device))
    d_pos = torch.from_numpy(pos).to(device)
    # the int8 + exponent form of the indexer rows is written when a row enters the cache (one row per sequence every
    # `ratio` tokens): built here once, like the cache contents themselves, outside the timed region
    n_rows = torch.full((B,), max_comp, dtype=torch.int32, device=device)
    layer.pack_index_rows(None, n_rows, max_comp)
    t0 = time.perf_counter()
    want_sel, want_out = orc.v4_decode_step_bf16(og, pos[:n_cpu], host["q"], host["kv_cache"], host["sink"], host["iq"],
                                                 host["iw"], host["ikv"])
    cpu_s = time.perf_counter() - t0
    layer.step(d_pos, q, iq, iw)
    torch.cuda.synchronize(device)
    assert np.array_equal(layer.sel[:n_cpu].cpu().numpy(), want_sel), "selection rows differ from the oracle"
    ok, worst = wl.attend_close(layer.out[:n_cpu].cpu().numpy(), want_out)
    assert ok, f"attention differs from the oracle: {worst}"

    sampler = ClockSampler(0)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    t_sel = t_att = 0.0
    for it in range(args.warmup + args.steps):
        if it == args.warmup:
            sampler.start()
            sampler.mark()
        ev[0].record()
        layer.select(d_pos, iq, iw)
        ev[1].record()
        layer.attend(q)
        ev[2].record()
        torch.cuda.synchronize(device)
        if it >= args.warmup:
            t_sel += ev[0].elapsed_time(ev[1])
            t_att += ev[1].elapsed_time(ev[2])
    sampler.mark()
    clocks = sampler.stop()
    assert not layer.refolded.any().item(), "the integer scorer handed spread rows to the ordered fold"
    t_sel, t_att = t_sel / args.steps, t_att / args.steps
    # end to end: pinned host inputs up, bf16 output down, every step
    h_in = [t.cpu().pin_memory() for t in (d_pos, q, iq, iw)]
    h_out = torch.empty(layer.out.shape, dtype=torch.uint16).pin_memory()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_e2e = max(3, args.steps // 4)
    e0.record()
    for _ in range(n_e2e):
        dp, dq, diq, diw = (t.to(device, non_blocking=True) for t in h_in)
        h_out.copy_(layer.step(dp, dq, diq, diw), non_blocking=True)
    e1.record()
    torch.cuda.synchronize(device)
    e2e_ms = e0.elapsed_time(e1) / n_e2e
    ms = t_sel + t_att
    peaks = {}
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    cols = g.window + g.index_topk
    att_bytes = B * (cols * g.head_dim * 2 + 2 * g.n_heads * g.head_dim * 2 + cols * 4)
    sel_bytes = B * (max_comp * (g.index_dim + 4) + g.index_heads * g.index_dim * 2 + max_comp * 8 + cols * 4)   # int8 rows + exps, scores w+r
    dom, dom_ms, dom_bytes = ("sparse_attend", t_att, att_bytes) if t_att >= t_sel else ("select_blocks", t_sel, sel_bytes)
    ach = dom_bytes / (dom_ms * 1e-3) / 1e9
    line = {"metric": "V4 sparse-attention decode layer-steps/s (batch x ctx)", "value": 1e3 / ms, "unit": "layer-steps/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, f32 accumulate; block scores exact f32 folds",
            "data": "synthetic",
            "config": {"workload": f"v4: batch {B} x context {w['ctx']}, {g.n_heads} heads x {g.head_dim}, ring {g.window} + "
                                   f"top-{g.index_topk} of {max_comp} ratio-{g.ratio} blocks, {g.index_heads}-head indexer, seed {w['seed']}",
                       "l2": "inputs larger than L2 (kv 285 MB; indexer rows 34 MB int8 + 67 MB bf16, only the int8 form is read)",
                       "index_rows": "int8 + block exponents, packed when a row enters the cache (untimed, like the cache fill)",
                       "stage_ms": {"select_blocks": t_sel, "sparse_attend": t_att}},
            "e2e": {"value": 1e3 / e2e_ms, "unit": "layer-steps/s",
                    "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in h_in)),
                    "d2h_bytes_per_step": int(h_out.numel() * 2)},
            "gpu_launches": args.steps * 3, "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": hbm_peak, "unit": "GB/s",
                         "frac": ach / hbm_peak,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch at this shape
                         # (profiles/ncu_full_v4_kernels_batch128_ctx8192.md)
                         "traffic": {"sparse_attend": 96.58e6, "select_blocks": 37.85e6}[dom],
                         "peak_source": "measured" if "hbm_gbs" in peaks else "fallback",
                         "stages": {"select_blocks": sel_bytes / (t_sel * 1e-3) / 1e9 / hbm_peak,
                                    "sparse_attend": att_bytes / (t_att * 1e-3) / 1e9 / hbm_peak}},
            "cpu_baseline": {"value": n_cpu / B / cpu_s, "unit": "layer-steps/s", "cores": orc.num_threads(), "kind": "port",
                             "sample": f"{n_cpu} of the {B} sequences, one step, scaled by {B}/{n_cpu}"}}
    print(json.dumps(line), flush=True)


def measure_cfg4(args, rank, world, device, steps, warmup):
    """Long-context decode, page-range sharded over the ranks (strong scaling: batch 4 x context 131,072 in total):
    a step = append the new token on the rank that owns the last page range, then rivoli_shard_step_paged - local
    selection, ncclAllGather of the candidates, exact global cut + local partial attention, ncclAllGather of the
    partials, merge. Timed on the device, MAX over ranks. Returns the result object (every rank) for rank 0 to print."""
    import torch
    import torch.distributed as dist
    from rivoli_b200 import shard
    w = dict(WORKLOADS["cfg4"])
    B, k = w["B"], w["top_k"]
    ctx_local = w["ctx"] // world
    g, layer, _ = build_layer(dict(w, ctx=ctx_local), device, w["seed"] * 100 + rank)   # ctx_local - 1 history tokens
    gen = torch.Generator(device=device)
    gen.manual_seed(w["seed"])                                                            # the step's inputs: same on every rank
    x = step_inputs(w, device, gen)
    last = rank == world - 1
    local_len = torch.full((B,), ctx_local if last else ctx_local - 1, dtype=torch.int32, device=device)
    offset = rank * (ctx_local - 1)
    new_pos = torch.full((B,), ctx_local - 1, dtype=torch.int32, device=device)
    comm = shard.ShardedDecodeStep.nccl_comm(rank, world)
    sh = shard.ShardedDecodeStep(layer, rank, world, comm)

    def step():
        if last:
            layer.append(x["latent"], x["index_key"], new_pos)
        return sh.step(x["index_q"], x["index_w"], x["q"], local_len)

    out = step()
    torch.cuda.synchronize(device)
    layer.check_status()
    # properties that need no oracle: the selected rows over all ranks number exactly k per sequence, each rank's are
    # ascending and inside its own range, and every rank holds the same merged output
    n_all = sh.n_mine.clone()
    dist.all_reduce(n_all)
    assert (n_all == k).all().item(), n_all.tolist()
    ra, nm = sh.rows_att.cpu().numpy().view(np.uint32).astype(np.int64), sh.n_mine.cpu().numpy()
    for b in range(B):
        r = ra[b, : nm[b]]
        assert np.all(np.diff(r) > 0) and (r.size == 0 or (r[0] >= 0 and r[-1] < int(local_len[b])))
    chk = out.view(torch.int16).to(torch.int64).sum().reshape(1)
    lo, hi = chk.clone(), chk.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    assert lo.item() == hi.item(), "ranks disagree on the merged output"
    for _ in range(warmup):
        step()

    def timed(fn, n):
        dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        dist.barrier()
        torch.cuda.synchronize(device)
        t = torch.tensor([e0.elapsed_time(e1) / n], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms = timed(step, steps)
    # the same kernels without the two collectives (buffers gathered once with torch.distributed): what is left of
    # the step is NCCL launch latency + transfer + the wait for the slowest rank
    cand = sh.candidates(x["index_q"], x["index_w"], local_len)
    all_cand = torch.empty(world * cand.numel(), dtype=torch.uint8, device=device)
    dist.all_gather_into_tensor(all_cand, cand)
    part = sh.cut_attend(all_cand, x["q"])
    all_part = torch.empty(world * part.numel(), dtype=torch.uint8, device=device)
    dist.all_gather_into_tensor(all_part, part)

    def local_only():
        if last:
            layer.append(x["latent"], x["index_key"], new_pos)
        sh.candidates(x["index_q"], x["index_w"], local_len)
        sh.cut_attend(all_cand, x["q"])
        sh.merge(all_part)

    for _ in range(3):
        local_only()
    ms_local = timed(local_only, steps)
    layer.check_status()
    dist.barrier()
    from rivoli_b200 import backend as be
    be.shard_nccl_comm_destroy(comm)
    per_seq = algorithmic_bytes(w)
    total = (per_seq["append"] + per_seq["index"] + per_seq["attend"]) * B
    res = {"metric": METRIC, "value": 1e3 / ms, "unit": "layer-steps/s", "n_gpus": world, "steps": steps, "warmup": warmup,
           "ms_per_step": ms, "scaling": "strong",
           "config": {"workload": f"cfg4: batch {B} x context {w['ctx']}, page-range sharded {world}-way "
                                  f"({ctx_local} tokens of every sequence per GPU), top-k {k}, seed {w['seed']}",
                      "call": "rivoli_shard_step_paged: tensor-core scorer + cluster selection + exact candidate scores, "
                              "ncclAllGather (candidates), global cut + partial attention, ncclAllGather (partials), merge",
                      "collectives_per_step": 2,
                      "bytes_per_rank_per_collective": [int(cand.numel()), int(part.numel())]},
           "ms_kernels_only": ms_local, "ms_collectives": ms - ms_local,
           "limiter": "two NCCL all-gathers of 33 KB / 265 KB per rank: launch latency and rank skew, not bandwidth; "
                      "the kernels run at batch 4 and are latency bound themselves",
           "gbs_per_gpu": total / (ms * 1e-3) / 1e9 / world,
           "self_check": "k rows in total per sequence, ascending inside every rank's range, identical merged output on every rank"}
    del sh, layer
    torch.cuda.empty_cache()
    return res


def run_cfg4(args):
    """`--workload cfg4` under torchrun with --gpus >= 2: the page-range sharded step alone; rank 0 prints one line."""
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    assert world >= 2 and world == args.gpus, "cfg4 is the page-range sharded case: launch it under torchrun with --gpus >= 2"
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)
    res = measure_cfg4(args, rank, world, device, steps=args.steps, warmup=max(args.warmup, 3))
    if rank == 0:
        res.update({"higher_is_better": True, "vs_baseline": None, "data": "synthetic",
                    "dtype": "fp8-e4m3 cache, bf16 activations, f32 accumulate", "gpu_launches": args.steps * 12})
        print(json.dumps(res), flush=True)
    dist.destroy_process_group()


def run_profile(args):
    import torch
    if args.profile == "proj":
        torch.cuda.set_device(0)
        print(time_projections(WORKLOADS[args.workload], torch.device("cuda", 0), steps=3))
        print("profile run ok: proj")
        return
    w = dict(WORKLOADS[args.workload])
    if args.batch:
        w["B"] = args.batch                                # a smaller case of the same shape for multi-pass captures
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g, layer, gen = build_layer(w, device, w["seed"])
    x = step_inputs(w, device, gen)
    row_pos = torch.full((w["B"],), w["ctx"] - 1, dtype=torch.int32, device=device)
    seq_len = torch.full((w["B"],), w["ctx"], dtype=torch.int32, device=device)
    layer.select(x["index_q"], x["index_w"], seq_len)      # rows for the attend-only mode
    for _ in range(3):
        if args.profile == "step":       # exactly what the bench's timed region launches
            layer.step(x["latent"], x["index_key"], x["index_q"], x["index_w"], x["q"], row_pos, seq_len)
        if args.profile == "select":
            layer.select(x["index_q"], x["index_w"], seq_len)
        if args.profile == "attend":
            layer.attend(x["q"])
    torch.cuda.synchronize(device)
    layer.check_status()
    print("profile run ok:", args.profile, args.workload)


def cpu_sample_state(w, n_seq, seed):
    """A bounded sample of the workload for the CPU arm: n_seq sequences of the same shape."""
    from oracle.workload import State
    return State(seed, n_seq, [w["ctx"]] * n_seq, n_heads=w["n_heads"], index_heads=w["index_heads"],
                 index_dim=w["index_dim"], page_tokens=w["page_tokens"], top_k=w["top_k"], pool_factor=1.25)


def cpu_baseline(w, seconds=12.0, n_seq=None):
    """Times the oracle (C restatement of the reference's host arithmetic, OpenMP) on a bounded
    sample of the same workload and scales to whole-batch layer-steps/s."""
    from oracle import oracle as orc
    orc.set_num_threads(len(os.sched_getaffinity(0)))      # all host threads this process may use
    n_seq = n_seq or max(1, min(w["B"], 8))
    st = cpu_sample_state(w, n_seq, w["seed"])
    t0 = time.perf_counter()
    reps = 0
    while True:
        st.oracle_step()
        reps += 1
        if time.perf_counter() - t0 > seconds or reps >= 50:
            break
    dt = (time.perf_counter() - t0) / reps
    per_seq = dt / n_seq
    return {"value": 1.0 / (per_seq * w["B"]), "unit": "layer-steps/s", "cores": orc.num_threads(),
            "kind": "port", "nproc": os.cpu_count(),
            "sample": f"{n_seq} of {w['B']} sequences of the same shape (ctx {w['ctx']}), {reps} repetitions, "
                      f"{dt:.3f} s per sample step; scaled by {w['B']}/{n_seq}"}


def run_reference(args):
    """The reference's own CPU arithmetic for this path (the oracle port: the reference is a
    Rust + HIP tree that cannot be compiled on this image), all host threads. A step = the layer-step on a bounded
    SAMPLE of the batch (8 of its sequences); `ms_per_step` is that sample step as measured, `sample_scale` the
    factor to the whole batch, `value` the whole-batch rate. The workload is the batch in total, whatever N is:
    the CPU arm is one host."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    from oracle import oracle as orc
    orc.set_num_threads(len(os.sched_getaffinity(0)))      # torchrun exports OMP_NUM_THREADS=1; rank 0 runs alone
    # bounded sample: about 11 ms of CPU work per cfg3 sequence; keep the whole run near two minutes
    per_seq_s = 0.011 * w["ctx"] / 16384
    warm = max(args.warmup, 3)
    n_seq = max(1, min(w["B"], 8, int(120.0 / max(1, args.steps + warm) / per_seq_s)))
    st = cpu_sample_state(w, n_seq, w["seed"])
    for _ in range(warm):
        st.oracle_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        st.oracle_step()
    dt = (time.perf_counter() - t0) / args.steps
    scale = w["B"] / n_seq
    value = 1.0 / (dt * scale)
    sample = (f"each step = {n_seq} of {w['B']} sequences of the same shape (ctx {w['ctx']}); value scaled by "
              f"{w['B']}/{n_seq}; one host, all threads")
    base = w["B"] // world
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "layer-steps/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": dt * 1e3, "sample_scale": scale,
            "ms_per_whole_batch_step": dt * scale * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32 (CPU)",
            "data": "synthetic",
            "config": config_of(args.workload, w, world, base if world > 1 else w["B"], "strong"),
            "cpu_baseline": {"value": value, "unit": "layer-steps/s", "cores": orc.num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": "layer-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    # rank 0 prints ONE JSON line on stdout: keep NCCL's version banner (NCCL_DEBUG=VERSION prints it there) out of it
    if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
        os.environ["NCCL_DEBUG"] = "WARN"
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3", choices=list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile", default=None, choices=["select", "attend", "step", "proj"],
                    help="build the workload, run 3 iterations of one stage (or the whole step) and exit: "
                         "the command line the profiles/ summaries were captured with")
    ap.add_argument("--layers", type=int, default=0, help="cfg5 only: number of layers (default 78)")
    ap.add_argument("--reps", type=int, default=0,
                    help="repetitions of the --steps loop inside the timed region (default: as many as make it 0.25 s long)")
    ap.add_argument("--batch", type=int, default=0,
                    help="with --profile only: sequences per GPU instead of the workload's own batch")
    args = ap.parse_args()
    if args.batch and not args.profile:
        ap.error("--batch is a --profile option; the bench always runs the workload's own batch")
    if args.profile:
        return run_profile(args)
    if args.workload == "cfg4":
        if args.impl == "reference":
            ap.error("cfg4 is a multi-GPU measurement of the CUDA arm")
        if args.steps == 400:
            args.steps = 100
        return run_cfg4(args)
    if args.workload == "v4":
        if args.impl == "reference" or args.gpus != 1:
            ap.error("the V4 workload is a one-GPU next-row measurement of the CUDA arm (its CPU arm is in the same line)")
        if args.steps == 400:
            args.steps = 2000            # 0.14 ms each: long enough for the clock sampler to see the timed region
        return run_v4(args)
    if args.workload == "cfg5":
        if args.impl == "reference":
            ap.error("the churn workload is a measurement of the CUDA arm (its parity check against the oracle is part of it)")
        if args.steps == 400:
            args.steps = 8               # token-steps of 78 layer-steps each
        return run_churn(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
