"""Benchmark of the routed-expert MoE hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode|prefill|fp8] [--bank affine2|fp4] [--batch B] [--distinct-layers NL]

decode (default): one step = one decoded token = LAYERS (40) MoE layer passes: per layer the sigmoid top-6 routing
tail with slot lookup and the routed experts (gate/up, SwiGLU, down, weighted sum) over the resident bank -- one
kernel launch per layer for one token.  The default workload is the 2-bit affine g128 bank, batch 1, 384 experts
per layer; the bank holds NL distinct layers (default 8, 30.6 GB) that the 40 passes cycle through with fresh
random routing, so the bytes a pass reads were last touched hundreds of MB ago (the working set is far larger than
L2).  The K-step timed region is repeated (at least five times, at least half a second in total) and the median
is reported.  Prints ONE JSON line (rank 0).

N > 1 shards the experts of every layer over the ranks (expert parallel, replicated input); the partial outputs
are summed through peer memory over NVLink in the tail of the expert kernel (`--reduce fused`, batch 1), by the
library's stand-alone peer-memory kernel (`--reduce peer`) or by an NCCL all-reduce (`--reduce nccl`); total work
is fixed ("strong" scaling).  Before timing, every rank checks a small sharded layer against the same layer on a
whole bank and the run stops with a non-zero exit code if they differ.
`--impl reference` times the CPU path (the numpy oracle port of the reference's arithmetic) on the host cores for
the same metric; the same function gives the `cpu_baseline` of the GPU arm.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

HIDDEN, INTER, EXPERTS, TOPK, LAYERS = 4096, 2880, 384, 6, 40
SWIGLU_LIMIT = 10.0
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# capture summarised under profiles/ (None until a capture exists for the workload).  Writes: the kernel's own
# 16 KB of output + 69 KB of hidden words; the capture's write counter also holds dirty lines of the bank fill that
# the launch's reads evict from L2 (1.7 MB / 14 MB in the two captures), which are not this kernel's traffic.
NCU_TRAFFIC_BYTES = {("affine2", 1, "fused"): 59829504 + 16384 + 69120, ("fp4", 1, "fused"): 112907264 + 16384 + 69120}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--bank", default="affine2", choices=["affine2", "fp4"])
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--workload", default="decode", choices=["decode", "prefill", "fp8", "head"],
                   help="prefill: one 4096-token chunk through one FP4 layer, Zipf(1.1) expert popularity (1 GPU); fp8: the FP8 trunk GEMV; head: the bf16 output head GEMV")
    p.add_argument("--tokens", type=int, default=4096, help="prefill chunk length")
    p.add_argument("--act", default="mxfp4", choices=["mxfp4", "bf16"],
                   help="prefill: activations quantised to MXFP4 per 32 (BASELINE config 3) or taken as bf16 with the reference's per-expert rounding points")
    p.add_argument("--experts", type=int, default=EXPERTS, help="prefill: experts in the layer (smaller = a case sized for profiling)")
    p.add_argument("--distinct-layers", type=int, default=8)
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-graph", action="store_true")
    p.add_argument("--reduce", default="fused", choices=["fused", "peer", "nccl"],
                   help="N > 1: how the ranks' partial layer outputs are summed (fused = in the tail of the expert kernel, "
                        "peer = the library's stand-alone peer-memory kernel, nccl = all_reduce)")
    p.add_argument("--repeats", type=int, default=0, help="repeats of the K-step timed region (0 = at least 5 and 0.5 s in total)")
    p.add_argument("--watchdog", type=int, default=0, help="dump all Python stacks and exit after this many seconds (0 = off)")
    return p.parse_args()


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ---- clocks ---------------------------------------------------------------------------------

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
            # nvidia-smi needs some tens of milliseconds to deliver its first line; the timed region is not much
            # longer, so wait for that line before the region starts
            t_end = time.time() + 2.0
            while not self.rows and time.time() < t_end:
                time.sleep(0.005)
            self.first = len(self.rows)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) < 9:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---- CPU arm --------------------------------------------------------------------------------

def cpu_layer_inputs(bank_kind: str, seed: int = 0):
    import numpy as np
    from oracle import configs, router

    rng = np.random.default_rng(seed)
    x = configs.round_bf16(rng.standard_normal((1, HIDDEN)).astype(np.float32))
    logits = rng.standard_normal(EXPERTS).astype(np.float32)
    inds, w, _ = router.route_tail(logits, np.zeros(EXPERTS, np.float32), np.arange(EXPERTS, dtype=np.int32)[None], 0, TOPK, 1.0,
                                   weights_bf16=False)
    make = configs.affine_expert if bank_kind == "affine2" else configs.fp4_expert
    experts = [make(np.random.default_rng([seed, int(e)]), HIDDEN, INTER) for e in inds]
    return x[0], w, experts


def cpu_layer_pass(bank_kind: str, x, w, experts, threads: int):
    """One MoE layer for one token on the host: the reference's CPU arithmetic (packed bytes ->
    dequant -> matvec -> SwiGLU -> down), experts spread over `threads` threads."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    from oracle import affine, fp4

    def one(i):
        e = experts[i]
        if bank_kind == "affine2":
            return affine.affine_expert_forward(x, e, bits=2, group_size=128, weight=w[i], swiglu_limit=SWIGLU_LIMIT)
        return fp4.expert_forward(x, e["w1.weight"], e["w1.scale"], e["w2.weight"], e["w2.scale"], e["w3.weight"], e["w3.scale"],
                                  weight=w[i], swiglu_limit=SWIGLU_LIMIT)

    if threads > 1:
        with ThreadPoolExecutor(max_workers=threads) as pool:
            outs = list(pool.map(one, range(len(experts))))
    else:
        outs = [one(i) for i in range(len(experts))]
    total = np.zeros(HIDDEN, np.float32)
    for o in outs:
        total = total + o
    return total


def cpu_threads() -> int:
    """Threads of the CPU arm: one per routed expert of a layer, as far as the host has cores."""
    return max(1, min(TOPK, os.cpu_count() or 1))


def time_cpu_token(bank_kind: str):
    """The CPU arm, used both as `cpu_baseline` and as `--impl reference`: ONE whole token really timed = LAYERS passes
    of a MoE layer (six routed experts from packed bytes: dequantise, three mat-vecs, SwiGLU, weighted sum) on
    `cpu_threads()` threads, after one untimed pass.  The passes reuse one layer's packed bytes (generating 240
    distinct experts on the host would take longer than the measurement; the cost is arithmetic, not memory).
    Returns (seconds per token, tok/s, threads, description)."""
    threads = cpu_threads()
    x, w, experts = cpu_layer_inputs(bank_kind)
    cpu_layer_pass(bank_kind, x, w, experts, threads)
    t0 = time.perf_counter()
    for _ in range(LAYERS):
        cpu_layer_pass(bank_kind, x, w, experts, threads)
    dt = time.perf_counter() - t0
    desc = (f"one token = {LAYERS} timed passes of one MoE layer (6 routed experts from packed bytes, numpy port of the reference's "
            f"arithmetic), {threads} threads, {dt:.1f} s; one untimed pass first; the passes reuse one layer's packed bytes")
    return dt, 1.0 / dt, threads, desc


def time_cpu_prefill(args):
    """The numpy oracle of the reference's prefill arithmetic on a bounded sample (a few tokens of the chunk:
    every routed row costs one expert dequantisation on the host).  Returns (tok/s, seconds, description)."""
    import numpy as np
    from oracle import configs, prefill

    sample, E = 4, args.experts
    rng = np.random.default_rng(0)
    ids, w = zipf_routing(rng, args.tokens, E, TOPK)
    ids, w = ids[:sample], w[:sample]
    x = configs.round_bf16(rng.standard_normal((sample, HIDDEN)).astype(np.float32))
    cache = {}

    def bank(e):
        if e not in cache:
            cache[e] = configs.fp4_expert(np.random.default_rng([0, int(e)]), HIDDEN, INTER)
        return cache[e]

    for e in set(ids.reshape(-1).tolist()):
        bank(e)                                   # weight generation is not part of the timed work
    t0 = time.perf_counter()
    prefill.moe_prefill_fp4(x, ids, w, bank, n_experts=E, swiglu_limit=SWIGLU_LIMIT, act="mxfp4")
    dt = time.perf_counter() - t0
    desc = f"{sample} tokens ({sample * TOPK} routed rows, {len(cache)} experts dequantised from packed bytes) of the {args.tokens}-token chunk, numpy"
    return sample / dt, dt / sample, desc


def run_reference_prefill(args):
    """CPU arm of the prefill workload."""
    E = args.experts
    tok_s, s_per_tok, desc = time_cpu_prefill(args)
    line = {
        "impl": "reference", "metric": "moe_prefill_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus, "steps": 1,
        "warmup": 0, "ms_per_step": s_per_tok * args.tokens * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"prefill expert-major MoE layer: FP4 E2M1/E8M0 bank, {E} experts, {args.tokens} tokens, top-{TOPK}, "
                               f"Zipf(1.1) expert popularity, hidden {HIDDEN}, inter {INTER}, activations MXFP4 per 32"},
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port", "sample": desc},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload == "prefill":
        return run_reference_prefill(args)
    dt, tok_s, threads, desc = time_cpu_token(args.bank)
    line = {
        "impl": "reference", "metric": "moe_decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": 1, "warmup": 0, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, {"parallelism": "cpu", "partial_sum": "none", "cuda_graph": False,
                                         "steps_note": f"--steps {args.steps} --warmup {args.warmup} asked; one token is timed (a token takes "
                                                       f"{dt:.0f} s on the host cores)"}),
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(args, extra):
    cfg = {
        "workload": ("decode MoE layer stack: " + ("2-bit affine g128 bank (fp16 scale+bias)" if args.bank == "affine2" else "FP4 E2M1/E8M0 bank")
                     + f", {EXPERTS} experts/layer, top-{TOPK} sigmoid routing, batch {args.batch}, hidden {HIDDEN}, inter {INTER}, "
                       f"{LAYERS} layer passes per token over {args.distinct_layers} distinct resident layers"),
        "bank": args.bank, "batch": args.batch, "layers_per_token": LAYERS, "distinct_layers": args.distinct_layers,
        "l2": "inputs larger than L2: each pass reads 6 random experts of a multi-GB bank; no flush needed",
    }
    if extra:
        cfg.update(extra)
    return cfg


# ---- GPU arm --------------------------------------------------------------------------------

def fill_bank(bank, gen):
    bank.fill_random(gen)


def _leave(world: int, closers=()) -> None:
    """End of a multi-rank run: all ranks stop together with nothing in flight, drop their peer mappings together
    (`closers`: objects with close()), and only then leave.  The process group is not torn down (captured graphs
    may still hold NCCL work, and tearing down with them alive blocks): the ranks exit at once after the barrier."""
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.synchronize()
        dist.barrier()
        for c in closers:
            if c is not None:
                c.close()
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def check_expert_parallel(cb, ep, dist, dev, rank, world, reduce_kind):
    """A small layer on this rank's shard with the cross-rank sum against the same layer on a whole bank, on every
    rank: True when every rank agrees within 2e-3 of the largest output and no status bit is set."""
    import torch

    hidden, inter, n_exp, k = 2048, 2816, 32, TOPK
    ok = True
    for kind in ("affine2", "fp4"):
        fmt = cb.affine_format(hidden, inter) if kind == "affine2" else cb.FP4_FORMAT
        whole = cb.SlabBank(fmt, hidden, inter, n_exp, layers=1, n_experts=n_exp, device=dev)
        whole.fill_random(torch.Generator(device=dev).manual_seed(77))
        lo, hi = ep.local_range(n_exp, rank, world)
        shard = cb.SlabBank(fmt, hidden, inter, max(hi - lo, 1), layers=1, n_experts=n_exp, device=dev)
        if hi > lo:
            shard.slab.copy_(whole.slab[lo:hi])
        table = ep.local_slot_table(1, n_exp, rank, world).to(dev)
        peer = ep.PeerLayer(hidden, dev) if reduce_kind == "fused" else None
        psum = ep.PeerSum(hidden, dev) if reduce_kind == "peer" else None
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        g = torch.Generator().manual_seed(3)
        for _ in range(4):
            x = torch.randn(hidden, generator=g).to(torch.bfloat16).to(dev)
            logits = torch.randn(n_exp, generator=g).to(dev)
            got = cb.moe_layer_decode(x, logits, shard, table=table, router="sigmoid", peer=peer, status=status)
            if psum is not None:
                got = psum(got, status=status)
            elif peer is None:
                dist.all_reduce(got)
            want = cb.moe_layer_decode(x, logits, whole, router="sigmoid")
            ok = ok and float((got - want).abs().max()) <= 2e-3 * float(want.abs().max())
        torch.cuda.synchronize(dev)
        ok = ok and int(status.item()) == 0
        for c in (peer, psum):
            if c is not None:
                c.close()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    import cachalot_b200 as cb
    from cachalot_b200 import _lib, ep

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    B, NL, K = args.batch, args.distinct_layers, TOPK
    fmt = cb.affine_format(HIDDEN, INTER) if args.bank == "affine2" else cb.FP4_FORMAT
    lo, hi = ep.local_range(EXPERTS, rank, world)
    n_local = hi - lo
    bank = cb.SlabBank(fmt, HIDDEN, INTER, NL * n_local, layers=NL, n_experts=EXPERTS, device=dev)
    table = ep.local_slot_table(NL, EXPERTS, rank, world).to(dev)
    fill_bank(bank, torch.Generator(device=dev).manual_seed(1234 + rank))

    # replicated inputs: identical seed on every rank
    P = 16
    g_in = torch.Generator().manual_seed(7)
    x_host = torch.randn((P, B, HIDDEN), generator=g_in).to(torch.bfloat16).pin_memory()
    logits_host = torch.randn((P, LAYERS, B, EXPERTS), generator=g_in).pin_memory()
    out_host = torch.empty((B, HIDDEN), dtype=torch.float32).pin_memory()
    x_pool, logits_pool = x_host.to(dev), logits_host.to(dev)
    x = x_pool[0].clone()
    logits = logits_pool[0].clone()
    out = torch.zeros((B, HIDDEN), dtype=torch.float32, device=dev)
    ws = torch.empty(max(_lib.lib.cachalot_moe_decode_workspace_bytes(bank.desc_ptr, B, K) + 4096, 1 << 20), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    slots_all = torch.empty((LAYERS, B, K), dtype=torch.int32, device=dev)
    w_all = torch.empty((LAYERS, B, K), dtype=torch.float32, device=dev)

    # cross-rank sum of the partial outputs.  No silent downgrade: what --reduce asks for either works and passes the
    # check against the unsharded layer, or the run stops with a non-zero exit code.
    peer_sum, peer_layer, reduce_kind = None, None, "none"
    if world > 1:
        reduce_kind = args.reduce if B == 1 or args.reduce != "fused" else "peer"   # the in-kernel exchange is the one-token kernel's
        if not check_expert_parallel(cb, ep, dist, dev, rank, world, reduce_kind):
            if rank == 0:
                print(f"expert-parallel check failed (--reduce {reduce_kind}): the sharded layer differs from the whole one",
                      file=sys.stderr, flush=True)
            torch.cuda.synchronize()
            os._exit(3)
        if reduce_kind == "fused":
            peer_layer = ep.PeerLayer(HIDDEN, dev)
        elif reduce_kind == "peer":
            peer_sum = ep.PeerSum(B * HIDDEN, dev)

    def token_step():
        for l in range(LAYERS):
            if B == 1:   # routing tail and experts in one launch
                cb.moe_layer_decode(x[0], logits[l][0], bank, layer=l % NL, topk=K, table=table, router="sigmoid", route_scale=1.0,
                                    swiglu_limit=SWIGLU_LIMIT, out=out[0], workspace=ws, status=status, peer=peer_layer)
            else:
                _, w, slots = cb.route_tail(logits[l], None, table, l % NL, K, 1.0, weights_bf16=False)
                cb.moe_forward(x, slots, w, bank, swiglu_limit=SWIGLU_LIMIT, out=out, workspace=ws, status=status)
            if peer_sum is not None:
                peer_sum(out.view(-1), status=status)
            elif world > 1 and peer_layer is None:
                dist.all_reduce(out)

    def phase_step(phase):
        for l in range(LAYERS):
            cb.moe_forward(x, slots_all[l], w_all[l], bank, swiglu_limit=SWIGLU_LIMIT, out=out, workspace=ws, status=status, phase=phase)

    stream = torch.cuda.Stream(device=dev)
    use_graph = not args.no_graph

    def make_runner(fn):
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            if not use_graph:
                return fn
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn()
            return g.replay

    run_token = make_runner(token_step)

    def barrier():
        # Drain this rank's stream BEFORE the NCCL barrier: its kernel runs on NCCL's own stream and does not wait for
        # work queued on `stream`.  A decode launch needs every SM (one CTA with all its shared memory per SM) and
        # waits for its peers inside the kernel, so an NCCL kernel that slips in between two queued launches on one
        # rank, while a peer's GPU is filled by a launch that waits for this rank, stalls both until the kernel's
        # bounded wait runs out.
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps, before=None, after=None):
        """CUDA-event time of `steps` calls on `stream`, max over ranks (ms)."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for i in range(steps):
                if before:
                    before(i)
                fn()
                if after:
                    after(i)
            e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def feed_device(i):
        x.copy_(x_pool[i % P], non_blocking=True)
        logits.copy_(logits_pool[i % P], non_blocking=True)

    def feed_host(i):
        x.copy_(x_host[i % P], non_blocking=True)
        logits.copy_(logits_host[i % P], non_blocking=True)

    def read_back(i):
        out_host.copy_(out, non_blocking=True)
        stream.synchronize()

    timed(run_token, args.warmup, feed_device)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    def repeated(before, after=None):
        """The K-step region repeated: at least five times and half a second in total, so that the clock sampler sees
        the GPU under load.  Returns (median, min, all) in ms per region; identical counts on every rank."""
        first = timed(run_token, args.steps, before, after)
        n = args.repeats if args.repeats > 0 else int(min(400, max(5, -(-500.0 // max(first, 1e-3)))))
        all_ms = sorted([first] + [timed(run_token, args.steps, before, after) for _ in range(n - 1)])
        return all_ms[len(all_ms) // 2], all_ms[0], all_ms

    ms, ms_min, ms_all = repeated(feed_device)
    ms_e2e, ms_e2e_min, _ = repeated(feed_host, read_back)
    clocks = sampler.stop() if rank == 0 else None

    # per-kernel durations: the same 40 passes with routing done beforehand
    with torch.cuda.stream(stream):
        distinct = 0
        for l in range(LAYERS):
            _, w, slots = cb.route_tail(logits[l], None, table, l % NL, K, 1.0, weights_bf16=False)
            slots_all[l], w_all[l] = slots, w
        stream.synchronize()
        for l in range(LAYERS):
            s = slots_all[l].reshape(-1)
            distinct += int(torch.unique(s[s >= 0]).numel())
    PER_TOKEN_MAX = 64      # up to this many tokens the library runs the single-launch kernel once per token
    fused = B <= PER_TOKEN_MAX   # gate/up, SwiGLU and down run as ONE launch per (layer, token)
    reps = max(3, args.steps // 2)
    if fused:
        run_layers = make_runner(lambda: phase_step(None))
        timed(run_layers, 2)
        ms_layer = timed(run_layers, reps) / (reps * LAYERS)
        ms_gu = ms_dn = None
    else:
        run_gu = make_runner(lambda: phase_step("gate_up"))
        run_dn = make_runner(lambda: phase_step("down"))
        timed(run_gu, 2)
        ms_gu = timed(run_gu, reps) / (reps * LAYERS)
        timed(run_dn, 2)
        ms_dn = timed(run_dn, reps) / (reps * LAYERS)
    st = int(status.item())

    if rank != 0:
        _leave(world, (peer_layer, peer_sum))
        return

    sizes = bank.tensor_sizes
    up_bytes = sum(v for n, v in sizes.items() if n.startswith(("w1", "w3")))
    dn_bytes = sum(v for n, v in sizes.items() if n.startswith("w2"))
    u_per_layer = distinct / LAYERS          # distinct experts this rank streams per pass (routing of pool entry 0)
    gu_alg = u_per_layer * up_bytes + B * HIDDEN * 2 + B * K * INTER * 4
    dn_alg = u_per_layer * dn_bytes + B * K * INTER * 4 + B * HIDDEN * 4
    peak, peak_kind = measured_peak()
    tok_s = B * args.steps / (ms * 1e-3)
    tok_s_e2e = B * args.steps / (ms_e2e * 1e-3)
    layer_bytes = u_per_layer * (up_bytes + dn_bytes) + B * HIDDEN * 2 + B * HIDDEN * 4
    hbm_gbs_token = layer_bytes * LAYERS * args.steps / (ms * 1e-3) / 1e9
    if fused and B == 1:
        # the timed region is LAYERS launches of this kernel per step (plus two small copies per token)
        us_launch = ms * 1e3 / (args.steps * LAYERS)
        gbs = layer_bytes / (us_launch * 1e-6) / 1e9
        roofline = {"kernel": "fused_decode_kernel (routing tail + W1,W3 dequant-GEMV + SwiGLU + W2 dequant-GEMV + sum over experts, one launch per layer)",
                    "bound": "hbm", "achieved": gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": gbs / peak,
                    "us_per_launch": us_launch, "algorithmic_bytes_per_launch": layer_bytes,
                    # the ncu capture is of a one-GPU launch; a rank of an expert-parallel run reads its share only
                    "traffic": NCU_TRAFFIC_BYTES.get((args.bank, B, "fused")) if world == 1 else None,
                    "us_per_launch_routing_done_beforehand": ms_layer * 1e3}
        launches = LAYERS * args.steps              # routing tail + experts = one launch per layer
    elif fused and args.bank == "fp4" and B >= int(os.environ.get("CACHALOT_GROUPED_MIN_ROWS", "8")):
        # FP4 bank from eight tokens up: rows grouped by expert, every distinct expert streamed once by the two grouped
        # block-scaled GEMMs (planning, residual quantiser, gate/up, down, combine: six launches after the routing one)
        us_layer = ms_layer * 1e3
        gbs = layer_bytes / (us_layer * 1e-6) / 1e9
        roofline = {"kernel": "grouped_mxf4_kernel x2 (gate/up, down) + planning, residual quantiser, combine; one layer, routing done beforehand",
                    "bound": "hbm", "achieved": gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": gbs / peak,
                    "us_per_launch": us_layer, "algorithmic_bytes_per_launch": layer_bytes, "distinct_experts_per_layer": u_per_layer,
                    "traffic": None}
        launches = 7 * LAYERS * args.steps
    elif fused:
        # a few tokens: per layer one routing launch and B launches of the single-token kernel (k experts each)
        launch_bytes = K * (up_bytes + dn_bytes) / max(world, 1) + HIDDEN * 2 + HIDDEN * 4
        us_launch = ms_layer * 1e3 / B
        gbs = launch_bytes / (us_launch * 1e-6) / 1e9
        roofline = {"kernel": "fused_decode_kernel, one launch per (layer, token) with the routing done beforehand",
                    "bound": "hbm", "achieved": gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": gbs / peak,
                    "us_per_launch": us_launch, "algorithmic_bytes_per_launch": launch_bytes, "traffic": None}
        launches = (1 + B) * LAYERS * args.steps
    else:
        gu_gbs = gu_alg / (ms_gu * 1e-3) / 1e9
        dn_gbs = dn_alg / (ms_dn * 1e-3) / 1e9
        roofline = {"kernel": "gate_up (W1,W3 dequant-GEMV + SwiGLU)", "bound": "hbm", "achieved": gu_gbs, "peak": peak,
                    "peak_kind": peak_kind, "unit": "GB/s", "frac": gu_gbs / peak, "us_per_launch": ms_gu * 1e3,
                    "algorithmic_bytes_per_launch": gu_alg, "traffic": NCU_TRAFFIC_BYTES.get((args.bank, B, "gate_up")),
                    "down": {"achieved": dn_gbs, "frac": dn_gbs / peak, "us_per_launch": ms_dn * 1e3,
                             "algorithmic_bytes_per_launch": dn_alg, "traffic": NCU_TRAFFIC_BYTES.get((args.bank, B, "down"))}}
        launches = 4 * LAYERS * args.steps          # routing tail, row grouping, gate/up, down per layer

    if peer_sum is not None:
        launches += LAYERS * args.steps             # the stand-alone peer-memory sum, one launch per layer
    line = {
        "metric": "moe_decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "ms_per_step_min": ms_min / args.steps, "repeats": len(ms_all),
        "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "int2xbf16->f32" if args.bank == "affine2" else "e2m1xbf16->f32", "data": "synthetic",
        "config": workload_config(args, {"parallelism": f"ep{world}", "partial_sum": reduce_kind, "cuda_graph": use_graph, "numerics_version": cb.NUMERICS_VERSION}),
        "clocks": clocks,
        "e2e": {"value": tok_s_e2e, "unit": "tok/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": int(x_host[0].numel() * 2 + logits_host[0].numel() * 4),
                "d2h_bytes_per_step": int(out_host.numel() * 4)},
        "gpu_launches": launches,
        "hbm": {"token_algorithmic_gbs": hbm_gbs_token, "frac_of_8tbs": hbm_gbs_token / 8000.0, "frac_of_peak": hbm_gbs_token / peak},
        "roofline": roofline,
        "status_word": st,
    }
    if world == 1 and not args.no_cpu_baseline:
        _, cpu_tok_s, threads, desc = time_cpu_token(args.bank)
        line["cpu_baseline"] = {"value": cpu_tok_s, "unit": "tok/s", "cores": threads, "kind": "port", "sample": desc}
    print(json.dumps(line), flush=True)
    _leave(world, (peer_layer, peer_sum))


# ---- prefill workload --------------------------------------------------------------------------

def zipf_routing(rng, tokens, n_experts, k, s=1.1):
    """k distinct experts per token with popularity ~ 1/rank**s under a seeded rank permutation
    (Gumbel top-k), weights = sigmoid of N(0,1) logits renormalised to sum 1."""
    import numpy as np

    p = 1.0 / np.arange(1, n_experts + 1) ** s
    p = p[rng.permutation(n_experts)]
    p /= p.sum()
    keys = np.log(p)[None, :] + rng.gumbel(size=(tokens, n_experts))
    ids = np.argsort(-keys, axis=1)[:, :k].astype(np.int32)
    w = 1.0 / (1.0 + np.exp(-rng.standard_normal((tokens, k))))
    return ids, (w / w.sum(1, keepdims=True)).astype(np.float32)


def run_prefill(args):
    """One step = one chunk of `--tokens` prompt tokens through one MoE layer: expert-major grouping,
    MXFP4 activation quantisation, the two grouped block-scaled FP4 GEMMs and the slot-ordered combine.
    N > 1: tokens and experts are both split over the ranks (expert parallel); rows travel to the owners of
    their experts as MXFP4 codes + scales and come back as bf16 rows (two variable all-to-alls over NCCL)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    import cachalot_b200 as cb
    from cachalot_b200 import ep

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    T, K, E = args.tokens, TOPK, args.experts
    lo, hi = ep.local_range(E, rank, world)
    bank = cb.SlabBank(cb.FP4_FORMAT, HIDDEN, INTER, max(hi - lo, 1), layers=1, n_experts=E, device=dev)
    if world > 1:
        bank.slot_table = ep.local_slot_table(1, E, rank, world).to(dev)
    bank.fill_random(torch.Generator(device=dev).manual_seed(1234 + rank))
    rng = np.random.default_rng(0)                      # the same routing on every rank; a rank takes its slice of the tokens
    P = 4
    t_lo, t_hi = rank * T // world, (rank + 1) * T // world
    Tl = t_hi - t_lo
    g_in = torch.Generator().manual_seed(7 + rank)
    x_host = torch.randn((P, Tl, HIDDEN), generator=g_in).to(torch.bfloat16).pin_memory()
    routes = [zipf_routing(rng, T, E, K) for _ in range(P)]
    ids_host = torch.stack([torch.from_numpy(r[0][t_lo:t_hi]) for r in routes]).pin_memory()
    w_host = torch.stack([torch.from_numpy(r[1][t_lo:t_hi]) for r in routes]).pin_memory()
    out_host = torch.empty((Tl, HIDDEN), dtype=torch.float32).pin_memory()
    x_pool, ids_pool, w_pool = x_host.to(dev), ids_host.to(dev), w_host.to(dev)
    x, ids, w = x_pool[0].clone(), ids_pool[0].clone(), w_pool[0].clone()
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.Stream(device=dev)
    result = [None]

    def step():
        if world > 1:
            result[0] = ep.ep_moe_prefill(x, ids, w, bank, n_experts=E, swiglu_limit=SWIGLU_LIMIT, status=status)
        else:
            result[0] = cb.moe_prefill_grouped(x, ids, w, bank, swiglu_limit=SWIGLU_LIMIT, mxfp4_act=1 if args.act == "mxfp4" else 0, status=status)

    def barrier():
        # Drain this rank's stream BEFORE the NCCL barrier: its kernel runs on NCCL's own stream and does not wait for
        # work queued on `stream`.  A decode launch needs every SM (one CTA with all its shared memory per SM) and
        # waits for its peers inside the kernel, so an NCCL kernel that slips in between two queued launches on one
        # rank, while a peer's GPU is filled by a launch that waits for this rank, stalls both until the kernel's
        # bounded wait runs out.
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(steps, host):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for i in range(steps):
                src = (x_host, ids_host, w_host) if host else (x_pool, ids_pool, w_pool)
                x.copy_(src[0][i % P], non_blocking=True)
                ids.copy_(src[1][i % P], non_blocking=True)
                w.copy_(src[2][i % P], non_blocking=True)
                step()
                if host:
                    out_host.copy_(result[0], non_blocking=True)
                    stream.synchronize()
            e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    timed(max(args.warmup, 3), False)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = timed(args.steps, False)
    ms_e2e = timed(args.steps, True)
    clocks = sampler.stop() if rank == 0 else None
    st = status.clone()
    if world > 1:
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
    if int(st.item()):
        raise RuntimeError(f"device status {int(st.item())}")
    if rank != 0:
        _leave(world)
        return
    touched = float(np.mean([len(set(r[0].reshape(-1).tolist())) for r in routes]))
    rows = T * K
    per_expert = 3 * (HIDDEN * INTER // 2 + HIDDEN * INTER // 32)
    act_bytes = T * HIDDEN * 2 + rows * (HIDDEN // 2 + HIDDEN // 32) * 2 + rows * (INTER // 2 + INTER // 32) * 2 + rows * HIDDEN * 2 * 2 + T * HIDDEN * 4
    alg = touched * per_expert + act_bytes
    us = ms * 1e3 / args.steps
    peak, which = measured_peak()
    flops = 6.0 * rows * INTER * HIDDEN
    cfg = {"workload": f"prefill expert-major MoE layer: FP4 E2M1/E8M0 bank, {E} experts, {T} tokens, top-{K}, Zipf(1.1) expert "
                       f"popularity, hidden {HIDDEN}, inter {INTER}, "
                       + ("activations MXFP4 per 32" if args.act == "mxfp4" else "activations bf16 (as four residual MXFP4 terms), g, u, h, y rounded to bf16"),
           "l2": f"inputs larger than L2: {E * 18.8e6 / 1e9:.1f} GB of expert weights are streamed per step",
           "parallelism": f"ep{world}"}
    if world > 1:
        remote = rows * (world - 1) / world               # expected share of rows whose expert lives on another rank
        cfg["exchange"] = {"dispatch_bytes": remote * (HIDDEN // 2 + HIDDEN // 32 + 4), "combine_bytes": remote * HIDDEN * 2,
                           "collective": "NCCL all_to_all_single (variable splits), twice per step"}
    line = {
        "metric": "moe_prefill_tok_per_s", "value": T / (us * 1e-6), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": us / 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp4 (E2M1 x E2M1, E8M0 block scales, f32 accumulate)", "data": "synthetic", "config": cfg,
        "roofline": {"bound": "hbm", "achieved": alg / us / 1e3, "peak": peak * world, "unit": "GB/s", "frac": alg / us / 1e3 / (peak * world),
                     "traffic": None, "peak_source": which, "kernel": "whole call: grouping, quantiser, gate/up GEMM, down GEMM, combine"
                     + (", exchanges" if world > 1 else ""), "tensor_tflops": flops / us / 1e6},
        "e2e": {"value": T / (ms_e2e * 1e-3 / args.steps), "unit": "tok/s", "h2d_bytes_per_step": Tl * HIDDEN * 2 + Tl * K * 8,
                "d2h_bytes_per_step": Tl * HIDDEN * 4},
        "gpu_launches": (10 if world == 1 else 9) * args.steps, "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        cpu_tok_s, _, desc = time_cpu_prefill(args)
        line["cpu_baseline"] = {"value": cpu_tok_s, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port", "sample": desc}
    print(json.dumps(line), flush=True)
    _leave(world)


# ---- FP8 trunk GEMV workload --------------------------------------------------------------------

FP8_SHAPES = ((12288, 4096), (4096, 8192))
FP8_BLOCK = 128
FP8_COPIES = 6      # distinct weight copies of each matrix a step walks through: 503 MB per step, four times L2


def fp8_alg_bytes(n, k, batch):
    return n * k + (n // FP8_BLOCK) * (k // FP8_BLOCK) * 4 + batch * k * 2 + batch * n * 2


def time_cpu_fp8(batch):
    """CPU arm of the FP8 workload: the numpy oracle (act_quant per 1x128 with fp32 scales, block-wise GEMV) over both
    whole matrices, one token at a time, repeated until about ten seconds have gone.  Returns (GB/s, description)."""
    import numpy as np
    from oracle import configs, fp8

    rng = np.random.default_rng(0)
    work = []
    for n, k in FP8_SHAPES:
        w, ws = configs.fp8_matrix(rng, n, k, FP8_BLOCK, "f32")
        work.append((configs.round_bf16(rng.standard_normal((1, k)).astype(np.float32)), w, ws))
    fp8.fp8_linear(work[0][0], work[0][1][:128], work[0][2][:1], block_size=FP8_BLOCK, scale_rule="f32")
    done, tokens, t0 = 0, 0, time.perf_counter()
    while time.perf_counter() - t0 < 10.0 and tokens < 64:
        for (n, k), (x, w, ws) in zip(FP8_SHAPES, work):
            fp8.fp8_linear(x, w, ws, block_size=FP8_BLOCK, scale_rule="f32")
            done += fp8_alg_bytes(n, k, 1)
        tokens += 1
    secs = time.perf_counter() - t0
    return done / secs / 1e9, f"{tokens} tokens through both whole matrices, one at a time (numpy port, block 128, fp32 scales), {secs:.1f} s"


def run_fp8(args):
    """One step = act_quant + GEMV over FP8_COPIES distinct copies of both trunk matrices ([12288,4096] and [4096,8192],
    E4M3 weights, fp32 scales per 128x128, activations quantised per 1x128), `--batch` tokens (1 or 32), replayed as
    one CUDA graph; value = algorithmic GB/s.  One GPU (the trunk GEMV is not sharded)."""
    import torch

    import cachalot_b200 as cb

    if args.impl == "reference" or int(os.environ.get("WORLD_SIZE", "1")) > 1 and int(os.environ.get("RANK", "0")) != 0:
        if int(os.environ.get("RANK", "0")) != 0:
            return
        gbs, desc = time_cpu_fp8(args.batch)
        print(json.dumps({"impl": "reference", "metric": "fp8_trunk_gemv_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": 1,
                          "warmup": 0, "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "e4m3",
                          "data": "synthetic", "config": {"workload": "FP8 E4M3 trunk GEMV with act_quant, block 128, fp32 scales"},
                          "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": os.cpu_count() or 1, "kind": "port", "sample": desc},
                          "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B = args.batch
    g = torch.Generator(device=dev).manual_seed(5)
    finite = torch.tensor([b for b in range(256) if (b & 0x7F) != 0x7F], dtype=torch.uint8, device=dev)
    mats = []
    for n, k in FP8_SHAPES:
        for _ in range(FP8_COPIES):
            w = finite[torch.randint(0, finite.numel(), (n, k), device=dev, generator=g)]
            ws = torch.rand((n // FP8_BLOCK, k // FP8_BLOCK), device=dev, generator=g) * 9e-3 + 1e-3
            mats.append((w, ws))
    P = 8
    gi = torch.Generator().manual_seed(3)
    x_host = [torch.randn((P, B, k), generator=gi).to(torch.bfloat16).pin_memory() for _, k in FP8_SHAPES]
    x_dev = [t.to(dev) for t in x_host]
    x = [t[0].clone() for t in x_dev]
    y = [torch.empty((B, n), dtype=torch.bfloat16, device=dev) for n, _ in FP8_SHAPES]
    y_host = [torch.empty((B, n), dtype=torch.bfloat16).pin_memory() for n, _ in FP8_SHAPES]
    codes = [torch.empty((B, k), dtype=torch.uint8, device=dev) for _, k in FP8_SHAPES]
    scales = [torch.empty((B, k // FP8_BLOCK), dtype=torch.float32, device=dev) for _, k in FP8_SHAPES]
    from cachalot_b200._lib import check, lib
    stream = torch.cuda.Stream(device=dev)

    def linear(mi, ci):
        w, ws = mats[mi * FP8_COPIES + ci]
        n, k = FP8_SHAPES[mi]
        check(lib.cachalot_fp8_linear(x[mi].data_ptr(), B, k, FP8_BLOCK, 1, codes[mi].data_ptr(), scales[mi].data_ptr(), w.data_ptr(),
                                      ws.data_ptr(), n, y[mi].data_ptr(), 1, stream.cuda_stream))

    def graph_of(fn):
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=stream):
                fn()
        return gr.replay

    step = graph_of(lambda: [linear(mi, ci) for ci in range(FP8_COPIES) for mi in range(2)])
    only = [graph_of(lambda mi=mi: [linear(mi, ci) for ci in range(FP8_COPIES)]) for mi in range(2)]

    def timed(fn, steps, host=False):
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for i in range(steps):
                for mi in range(2):
                    x[mi].copy_((x_host if host else x_dev)[mi][i % P], non_blocking=True)
                fn()
                if host:
                    for mi in range(2):
                        y_host[mi].copy_(y[mi], non_blocking=True)
                    stream.synchronize()
            e1.record(stream)
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1)

    timed(step, max(args.warmup, 3))
    sampler = ClockSampler(0)
    sampler.start()
    first = timed(step, args.steps)
    n_rep = args.repeats if args.repeats > 0 else int(min(400, max(5, -(-500.0 // max(first, 1e-3)))))
    all_ms = sorted([first] + [timed(step, args.steps) for _ in range(n_rep - 1)])
    ms = all_ms[len(all_ms) // 2]
    ms_e2e = sorted(timed(step, args.steps, True) for _ in range(5))[2]
    clocks = sampler.stop()
    per = [sorted(timed(only[mi], args.steps) for _ in range(5))[2] / (args.steps * FP8_COPIES) * 1e3 for mi in range(2)]  # us per linear
    # parity of what was timed: the last copy of each matrix against the oracle on a few rows
    import numpy as np
    from oracle import fp8 as ofp8
    for mi in range(2):
        w, ws = mats[mi * FP8_COPIES + FP8_COPIES - 1]
        rows = slice(0, 256)
        want = ofp8.fp8_linear(x[mi].float().cpu().numpy(), w[rows].cpu().numpy(), ws[:2].cpu().numpy(), block_size=FP8_BLOCK, scale_rule="f32")
        got = y[mi][:, rows].float().cpu().numpy()
        err = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
        if not err < 2 ** -7:
            print(f"fp8 workload: output differs from the oracle ({err:.3e})", file=sys.stderr, flush=True)
            sys.exit(3)
    alg = [fp8_alg_bytes(n, k, B) for n, k in FP8_SHAPES]
    step_bytes = FP8_COPIES * sum(alg)
    peak, which = measured_peak()
    gbs = step_bytes * args.steps / (ms * 1e-3) / 1e9
    line = {
        "metric": "fp8_trunk_gemv_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "ms_per_step_min": all_ms[0] / args.steps, "repeats": len(all_ms), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
        "config": {"workload": f"FP8 E4M3 trunk GEMV with act_quant: [12288,4096] and [4096,8192], fp32 scales per 128x128, activations per 1x128, "
                               f"batch {B}; a step = {FP8_COPIES} distinct copies of both matrices", "batch": B,
                   "l2": f"inputs larger than L2: a step streams {step_bytes / 1e6:.0f} MB of distinct weights", "cuda_graph": True},
        "clocks": clocks,
        "e2e": {"value": step_bytes * args.steps / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(sum(B * k * 2 for _, k in FP8_SHAPES)),
                "d2h_bytes_per_step": int(sum(B * n * 2 for n, _ in FP8_SHAPES))},
        "gpu_launches": 4 * FP8_COPIES * args.steps,
        "roofline": {"kernel": "fp8_gemv_stream_kernel (+ act_quant_kernel in front of it)", "bound": "hbm", "achieved": gbs, "peak": peak,
                     "peak_kind": which, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                     "per_matrix": [{"shape": list(FP8_SHAPES[mi]), "us_per_linear": per[mi], "algorithmic_bytes": alg[mi],
                                     "achieved": alg[mi] / per[mi] / 1e3, "frac": alg[mi] / per[mi] / 1e3 / peak} for mi in range(2)]},
    }
    if not args.no_cpu_baseline:
        cg, desc = time_cpu_fp8(B)
        line["cpu_baseline"] = {"value": cg, "unit": "GB/s", "cores": os.cpu_count() or 1, "kind": "port", "sample": desc}
    print(json.dumps(line), flush=True)


HEAD_SHAPE = (129280, 5120)   # the reference's output head (model/bf16_gemv_metal.py:4-8)


def run_head(args):
    """One step = one bf16-weight fp32 GEMV over the output head ([129280,5120] bf16 = 1.32 GB, ten times L2),
    `--batch` activation rows (1..8) sharing the pass; value = algorithmic GB/s.  One GPU (not sharded)."""
    import numpy as np
    import torch

    import cachalot_b200 as cb
    from cachalot_b200._lib import check, lib
    n, k = HEAD_SHAPE
    B = max(1, min(8, args.batch))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(11)
    w = (torch.randn((n, k), device=dev, generator=g) * 0.02).to(torch.bfloat16)
    P = 8
    x_host = torch.randn((P, B, k), generator=torch.Generator().manual_seed(3)).pin_memory()
    x_dev, x = x_host.to(dev), torch.empty((B, k), device=dev)
    y, y_host = torch.empty((B, n), device=dev), torch.empty((B, n)).pin_memory()
    stream = torch.cuda.Stream(device=dev)

    def timed(steps, host=False):
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for i in range(steps):
                x.copy_((x_host if host else x_dev)[i % P], non_blocking=True)
                check(lib.cachalot_bf16_gemv_f32(x.data_ptr(), B, w.data_ptr(), n, k, y.data_ptr(), stream.cuda_stream))
                if host:
                    y_host.copy_(y, non_blocking=True)
                    stream.synchronize()
            e1.record(stream)
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1)

    timed(max(args.warmup, 3))
    sampler = ClockSampler(0)
    sampler.start()
    all_ms = sorted(timed(args.steps) for _ in range(max(5, args.repeats)))
    ms = all_ms[len(all_ms) // 2]
    ms_e2e = sorted(timed(args.steps, True) for _ in range(5))[2]
    clocks = sampler.stop()
    # parity of what was timed: sampled rows against a float64 product
    want = (w[::1009].double() @ x.double().T).T.float()
    err = float((y[:, ::1009] - want).abs().max() / want.abs().max())
    if not err < 1e-5:
        print(f"head workload: output differs from the float64 product ({err:.3e})", file=sys.stderr, flush=True)
        sys.exit(3)
    alg = n * k * 2 + B * k * 4 + B * n * 4
    peak, which = measured_peak()
    gbs = alg * args.steps / (ms * 1e-3) / 1e9
    line = {
        "metric": "bf16_head_gemv_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "ms_per_step_min": all_ms[0] / args.steps, "repeats": len(all_ms), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x f32 -> f32", "data": "synthetic",
        "config": {"workload": f"bf16-weight fp32 GEMV over the output head [{n},{k}], batch {B}", "batch": B,
                   "l2": f"inputs larger than L2: a step streams {alg / 1e6:.0f} MB"},
        "clocks": clocks,
        "e2e": {"value": alg * args.steps / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": B * k * 4, "d2h_bytes_per_step": B * n * 4},
        "gpu_launches": args.steps,
        "roofline": {"kernel": "bf16_gemv_kernel", "bound": "hbm", "achieved": gbs, "peak": peak, "peak_kind": which, "unit": "GB/s",
                     "frac": gbs / peak, "us_per_launch": ms / args.steps * 1e3, "algorithmic_bytes_per_launch": alg, "traffic": None},
    }
    if not args.no_cpu_baseline:
        from oracle import bf16_gemv as obg
        bits = w[:8192].cpu().view(torch.int16).numpy().view(np.uint16)
        xs = x[:1].cpu().numpy()
        obg.bf16_gemv_f32(xs, bits[:64])
        t0 = time.perf_counter()
        obg.bf16_gemv_f32(xs, bits)
        secs = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 8192 * k * 2 / secs / 1e9, "unit": "GB/s", "cores": os.cpu_count() or 1, "kind": "port",
                                "sample": f"8192 of the {n} rows, one activation row, numpy (widen to float64, matmul), {secs:.2f} s"}
    print(json.dumps(line), flush=True)


def run_reference_gemv(args):
    """CPU arm of the two GEMV workloads: the numpy oracle on the host cores, a bounded sample."""
    import numpy as np

    if args.workload == "fp8":
        gbs, desc = time_cpu_fp8(max(1, args.batch))
        metric, cfg = "fp8_trunk_gemv_gbs", "FP8 E4M3 trunk GEMV with act_quant: [12288,4096] and [4096,8192], fp32 scales per 128x128"
    else:
        from oracle import bf16_gemv as obg
        n, k = HEAD_SHAPE
        rng = np.random.default_rng(0)
        bits = (rng.standard_normal((8192, k)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        xs = rng.standard_normal((1, k)).astype(np.float32)
        obg.bf16_gemv_f32(xs, bits[:64])
        t0 = time.perf_counter()
        obg.bf16_gemv_f32(xs, bits)
        secs = time.perf_counter() - t0
        gbs, desc = 8192 * k * 2 / secs / 1e9, f"8192 of the {n} rows, one activation row, numpy (widen to float64, matmul), {secs:.2f} s"
        metric, cfg = "bf16_head_gemv_gbs", f"bf16-weight fp32 GEMV over the output head [{n},{k}]"
    line = {"impl": "reference", "metric": metric, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": 1, "warmup": 0,
            "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": cfg, "batch": max(1, args.batch)},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": os.cpu_count() or 1, "kind": "port", "sample": desc},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    if args.watchdog > 0:
        import faulthandler

        faulthandler.dump_traceback_later(args.watchdog, exit=True)
    if args.impl == "reference" and args.workload in ("fp8", "head"):
        if int(os.environ.get("RANK", "0")) == 0:
            run_reference_gemv(args)
    elif args.workload == "fp8":
        run_fp8(args)
    elif args.workload == "head":
        run_head(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload == "prefill":
        run_prefill(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
