#!/usr/bin/env python
"""Benchmark of the TurboQuant KV-cache hot path on B200.

One "step" is the fused decode step of the batched ragged workload: the scatter
write of one new token per sequence into the paged 4-bit cache, followed by paged
split-K decode attention (export of per-split partials + log-sum-exp combine).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

prints ONE JSON line (rank 0). `value` is the KV-cache bytes the decode reads per
second (the reference's own accounting: ctx * H_kv * (d + 8) bytes per sequence),
summed over all ranks, inputs resident in HBM; `e2e` is the same metric through the
host-buffer call path with the per-step host<->device copies inside the timed region.
With N > 1 (under torchrun) every rank runs its own batch -- sequences are
independent, so there is no collective on the data path -- and the time is the max
over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The batched ragged decode configuration (64 sequences, 32 query / 8 KV heads,
# head size 128, context lengths uniform in [512, 32768], 16-token pages).
BATCH, HQ, HKV, D, S = 64, 32, 8, 128, 16
CTX_LO, CTX_HI = 512, 32768
WORKLOAD = "ragged_decode_b64_h32x8_d128_ctx512-32768_fused_step"
# The long-context configuration: 128 sequences of 65536 tokens in the whole job.
LONG_BATCH, LONG_CTX = 128, 65536
LONG_WORKLOAD = "long_context_decode_b128_h32x8_d128_ctx65536_fused_step"


def kv_bytes(ctx_lens) -> int:
    from ascend_micro_harness_b200.sharding import kv_bytes as _kv
    return _kv(ctx_lens, HKV, D)


def context_lengths(seed: int, batch: int = BATCH, lo: int = CTX_LO, hi: int = CTX_HI):
    rng = np.random.default_rng(seed)
    return rng.integers(lo, hi + 1, size=batch).astype(np.int64)


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, f"/tmp/tq_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.index)], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                cols = [c.strip() for c in line.split(",")]
                if len(cols) < 7:
                    continue
                try:
                    sm.append(float(cols[0]))
                    smax.append(float(cols[1]))
                except ValueError:
                    continue
                for n, c in zip(names, cols[3:7]):
                    if c == "Active":
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------- our arm
def build_workload(torch, dev, seed, ctx=None):
    """Seeded synthetic paged cache in HBM, generated directly in quantised form."""
    ctx = context_lengths(seed) if ctx is None else ctx
    B = len(ctx)
    pages_per_seq = (ctx + 1 + S - 1) // S           # room for the token the step writes
    total_pages = int(pages_per_seq.sum()) + 64
    max_blocks = int(pages_per_seq.max())
    rng = np.random.default_rng(seed + 1)
    perm = rng.permutation(total_pages)
    tables = np.zeros((B, max_blocks), np.int32)
    at = 0
    for b in range(B):
        n = int(pages_per_seq[b])
        tables[b, :n] = perm[at:at + n]
        at += n
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    nbytes = total_pages * HKV * S * D // 2
    key_cache = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=dev, generator=g)
    value_cache = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=dev, generator=g)
    inv = float(np.float32(1.0) / np.sqrt(np.float32(D)))
    e = torch.randint(0, 3, (2 * total_pages * HKV * S,), device=dev, generator=g)
    scale_cache = (torch.ldexp(torch.ones_like(e, dtype=torch.float32), e - 2) * inv).contiguous()
    signs = torch.where(torch.rand(D, device=dev, generator=g) < 0.5, -1.0, 1.0).float()
    # per-step host inputs (pinned): one new token per sequence, the query, slots, lengths
    hk = torch.randn((B, HKV * D), generator=torch.Generator().manual_seed(seed)).bfloat16().pin_memory()
    hv = torch.randn((B, HKV * D), generator=torch.Generator().manual_seed(seed + 2)).bfloat16().pin_memory()
    hq = torch.randn((B, HQ, D), generator=torch.Generator().manual_seed(seed + 3)).bfloat16().pin_memory()
    slots = np.array([tables[b, ctx[b] // S] * S + ctx[b] % S for b in range(B)], np.int32)
    hslots = torch.from_numpy(slots).pin_memory()
    hctx = torch.from_numpy((ctx + 1).astype(np.int32)).pin_memory()
    return dict(ctx=ctx + 1, total_pages=total_pages, max_blocks=max_blocks, inv=inv,
                key_cache=key_cache, value_cache=value_cache, scale_cache=scale_cache, signs=signs,
                tables=torch.from_numpy(tables).to(dev), hk=hk, hv=hv, hq=hq, hslots=hslots,
                hctx=hctx, tables_np=tables)


def run_ours(args):
    import torch
    import ascend_micro_harness_b200 as tq
    from ascend_micro_harness_b200.sharding import aggregate

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the engine has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    tq.load_library()

    # The job's batch is BATCH sequences per GPU, generated as one stream (rank r's seed adds the
    # r-th block of BATCH lengths, so one GPU sees the same batch at every N) and dealt to the
    # GPUs by the sharding helper: longest first to the lightest GPU, BATCH sequences each.
    from ascend_micro_harness_b200.sharding import partition_sequences
    long_ctx = args.workload == "long"
    if long_ctx:
        # 128 sequences of 65536 tokens in all, dealt round robin: the batch per GPU shrinks as N grows
        if LONG_BATCH % world != 0:
            raise SystemExit("bench.py --workload long: the GPU count must divide 128")
        ctx_all = np.full(LONG_BATCH, LONG_CTX, np.int64)
        mine = partition_sequences(ctx_all, world, "round_robin")[rank]
    else:
        ctx_all = np.concatenate([context_lengths(4 + r) for r in range(world)])
        mine = partition_sequences(ctx_all, world, "lpt_equal")[rank] if world > 1 else list(range(BATCH))
    w = build_workload(torch, dev, seed=4 + rank, ctx=ctx_all[np.asarray(mine)])
    nseq = len(mine)   # sequences on this GPU
    ctx = w["ctx"]
    splits = tq.choose_splits(nseq, HKV, S, int(ctx.max()),
                              torch.cuda.get_device_properties(dev).multi_processor_count)
    ws = torch.zeros(tq.decode_workspace_floats(nseq, HQ, HKV, D, splits), dtype=torch.float32, device=dev)
    out = torch.zeros((nseq, HQ, D), dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # Per-step host inputs live in ONE pinned staging buffer (k | v | q | slots | lens) with a
    # device twin, so the end-to-end step is one host->device copy, the three launches and one
    # device->host copy of the output.
    parts = [w["hk"], w["hv"], w["hq"], w["hslots"], w["hctx"]]
    sizes = [(t.numel() * t.element_size() + 255) // 256 * 256 for t in parts]
    host_in = torch.empty(sum(sizes), dtype=torch.uint8).pin_memory()
    dev_in = torch.empty(sum(sizes), dtype=torch.uint8, device=dev)
    views, at = [], 0
    for t, n in zip(parts, sizes):
        nb = t.numel() * t.element_size()
        host_in[at:at + nb].copy_(t.reshape(-1).view(torch.uint8))
        views.append(dev_in[at:at + nb].view(t.dtype).view(t.shape))
        at += n
    dev_in.copy_(host_in)
    dk, dv, dq, dslots, dctx = views
    hout = torch.empty((nseq, HQ, D), dtype=torch.bfloat16).pin_memory()
    geom = dict(num_kv_heads=HKV, head_size=D, block_size=S, num_blocks=w["total_pages"],
                inv_sqrt_len=w["inv"])
    scale = float(1.0 / np.sqrt(D))

    def scatter():
        tq.reshape_scatter(dk, dv, w["key_cache"], w["value_cache"], w["scale_cache"], dslots,
                           w["signs"], None, num_requests=nseq, status=status, **geom)

    def export():
        tq.decode_splitk_export(dq, w["key_cache"], w["value_cache"], w["scale_cache"], w["tables"],
                                dctx, w["signs"], ws, num_heads=HQ, splits=0,
                                softmax_scale=scale, max_context_hint=int(ctx.max()), status=status,
                                **geom)

    def combine():
        tq.splitk_combine(ws, w["signs"], None, out, items=nseq * HKV, rows=HQ // HKV,
                          rows_stride=HQ // HKV, head_size=D, splits=splits,
                          output_stage=tq.OUT_UNROTATED, inv_sqrt_len=w["inv"])

    def step():
        scatter()
        export()
        combine()

    def e2e_body():
        dev_in.copy_(host_in, non_blocking=True)
        step()
        hout.copy_(out, non_blocking=True)

    # The end-to-end step as a serving loop issues it: host->device copy of the step's inputs,
    # the three launches and the device->host copy of the output captured once as a CUDA graph
    # (the library neither allocates nor synchronises, so its launches are capturable), then one
    # graph launch and one stream synchronisation per step.
    e2e_graph = None
    try:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            e2e_body()                       # warm-up on the capture stream
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph):
            e2e_body()
    except Exception as exc:                 # capture refused: issue the five calls one by one
        print(f"bench.py: CUDA graph capture of the end-to-end step failed ({exc}); eager calls", file=sys.stderr)
        e2e_graph = None

    def e2e_step():
        if e2e_graph is not None:
            e2e_graph.replay()
        else:
            e2e_body()
        torch.cuda.current_stream().synchronize()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        barrier()
        ms, _ = aggregate(ev0.elapsed_time(ev1), 0, dist, dev)   # max over ranks
        return ms

    for _ in range(max(args.warmup, 3)):
        step()
    # The timed steps are issued as replays of one captured step (scatter, export, combine): one
    # host call per step, so a short run is not dominated by the first step's launch gaps.
    step_issue = step
    try:
        torch.cuda.synchronize()
        step_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(step_graph):
            step()
        step_issue = step_graph.replay
        step_issue()
    except Exception as exc:
        print(f"bench.py: CUDA graph capture of the step failed ({exc}); eager launches", file=sys.stderr)
        step_issue = step
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_total = timed(step_issue, args.steps)
    for _ in range(2):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps)

    # the dominant kernel on its own, CUDA events on the launching stream
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(args.steps)]
    barrier()
    step()   # one untimed step: the first launches after a barrier start on an idle GPU
    for a, b in evs:
        scatter()
        a.record()
        export()
        b.record()
        combine()
    barrier()
    kernel_ms = statistics.median(a.elapsed_time(b) for a, b in evs)
    clocks = sampler.stop() if rank == 0 else None
    assert int(status.item()) == 0, f"device status word {int(status.item())}"

    my_bytes = kv_bytes(ctx)
    _, total_bytes = aggregate(0.0, my_bytes, dist, dev)

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        ms_step = ms_total / args.steps
        value = total_bytes / (ms_step * 1e-3) / 1e9
        achieved = my_bytes / (kernel_ms * 1e-3) / 1e9
        h2d = host_in.numel()
        extra = side_measurements(torch, tq, dev, args)
        line = {
            "metric": "splitk_4bit_decode_kv_hbm_gbs", "value": round(value, 1), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "strong" if long_ctx else "weak",
            "vs_baseline": None, "dtype": "int4 codes; QK s8 x s8 -> s32, PV f16 x f16 -> f32", "data": "synthetic",
            "config": {"workload": LONG_WORKLOAD if long_ctx else WORKLOAD, "batch_per_gpu": nseq, "q_heads": HQ, "kv_heads": HKV,
                       "head_dim": D, "page_tokens": S, "splits": int(splits),
                       "kv_bytes_per_gpu": my_bytes,
                       "l2": "inputs larger than L2 (%.2f GB of cache read per step)" % (my_bytes / 1e9),
                       "parallelism": f"{nseq * world} sequences dealt to {world} GPU(s) "
                                      + ("round robin" if long_ctx else "by total context (longest first)")
                                      + f", {nseq} each, no collective"},
            "decode_us_per_step": round(kernel_ms * 1e3, 1),
            "e2e": {"value": round(total_bytes / (ms_e2e / args.steps * 1e-3) / 1e9, 1),
                    "unit": "GB/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(hout.numel() * hout.element_size()),
                    "ms_per_step": round(ms_e2e / args.steps, 4),
                    "issue": "one CUDA graph (copy in, 3 kernels, copy out) + stream sync per step"
                             if e2e_graph is not None else "5 calls + stream sync per step"},
            "gpu_launches": 3 * args.steps,
            "issue": "one CUDA graph replay (3 kernels) per step" if step_issue is not step else "3 launches per step",
            "roofline": {"kernel": "tq_decode_partial_kernel<128>", "bound": "hbm",
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}",
                         "traffic": DECODE_TRAFFIC_BYTES_PER_ALGORITHMIC_BYTE and
                         int(my_bytes * DECODE_TRAFFIC_BYTES_PER_ALGORITHMIC_BYTE)},
            "clocks": clocks,
            "extra": extra,
        }
        if world == 1:
            line["cpu_baseline"] = cpu_baseline_decode(w, args, sample=2 if long_ctx else nseq)
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# dram bytes (read + write) per algorithmic byte of the decode export kernel, from the ncu
# capture of the small ragged case (profiles/decode_partial_kernel_small_ragged.md):
# 224.52 MB + 7.53 MB over 223.39 MB. Traffic grows with the cache bytes read, so the full
# launch is scaled by its algorithmic bytes.
DECODE_TRAFFIC_BYTES_PER_ALGORITHMIC_BYTE = 1.0387


def side_measurements(torch, tq, dev, args):
    """The other two parts of the metric: reshape tokens/s on a scaled bf16 prefill and
    decode us/step at batch 1, context 4096 for split-K 2/4/8/16."""
    out = {}
    # --- reshape_and_cache, bf16, 8 KV heads x 128, 256 Ki tokens (inputs 1 GiB > L2)
    T, H = 262144, 8
    g = torch.Generator(device=dev)
    g.manual_seed(2)
    k = torch.randn((T, H * D), device=dev, generator=g, dtype=torch.float32).bfloat16()
    v = torch.randn((T, H * D), device=dev, generator=g, dtype=torch.float32).bfloat16()
    P = T // S
    kc = torch.empty(P * H * S * D // 2, dtype=torch.uint8, device=dev)
    vc = torch.empty_like(kc)
    sc = torch.empty(2 * P * H * S, dtype=torch.float32, device=dev)
    perm = torch.randperm(P, device=dev, generator=g)
    slots = (perm[:, None] * S + torch.arange(S, device=dev)[None, :]).reshape(-1).int().contiguous()
    signs = torch.where(torch.rand(D, device=dev, generator=g) < 0.5, -1.0, 1.0).float()
    inv = float(np.float32(1.0) / np.sqrt(np.float32(D)))

    def reshape():
        tq.reshape_and_cache(k, v, kc, vc, sc, slots, signs, num_kv_heads=H, head_size=D,
                             block_size=S, num_blocks=P, inv_sqrt_len=inv)
    for _ in range(3):
        reshape()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    reps = max(args.steps, 5)
    for _ in range(reps):
        reshape()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    nbytes = 2 * T * H * D * 2 + 2 * T * H * D // 2 + 2 * T * H * 4
    peak, _ = measured_peak_gbs()
    out["reshape_bf16"] = {"workload": "bf16 prefill 262144 tokens x 8 KV heads x 128, permuted pages",
                           "tokens_per_s": round(T / (ms * 1e-3)), "ms": round(ms, 4),
                           "gbs": round(nbytes / (ms * 1e-3) / 1e9, 1),
                           "frac_of_hbm_peak": round(nbytes / (ms * 1e-3) / 1e9 / peak, 4)}
    del k, v, kc, vc, sc
    return out


def _use_reference_geometry():
    """Switch the module's workload constants to head size 256 with 16 query / 4 KV heads."""
    global D, HQ, HKV
    D, HQ, HKV = 256, 16, 4


def run_profile_case(args):
    """A small case of one kernel for an ncu capture: inputs larger than L2 but well under
    a GB on the device, two warm-up launches and three captured ones.
      decode  : 64 sequences x 2048..4096 tokens (about 0.2 GB of cache)
      decode_d256 : the same at head size 256 with 16 query / 4 KV heads
      config3 : batch 1, context 4096, split-K swept over 1/2/4/8/16/auto: prints microseconds per decode
      reshape : bf16 prefill of 65536 tokens x 8 KV heads x 128 (0.27 GB)
      reshape_a8 : the same prefill with int8 activations (0.13 GB)
      lm_decode  : the Lloyd-Max cache variant, 64 sequences x 2048..4096 tokens, 2 splits
      lm_reshape : its bf16 writer on the 65536-token prefill
      scatter    : the 1-token-per-sequence writer of a 64-sequence decode step
      nz_import  : the KV4/FP8 NZ-tiled importer, 2048 pages x 128 slots x 4 heads (0.27 GB in)"""
    import torch
    import ascend_micro_harness_b200 as tq
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if args.profile == "config3":
        # batch 1, context 4096, shuffled table: microseconds per decode (export + combine) for
        # explicit split counts and for the library's own choice, L2 flushed before every call
        ctx_len, P = 4096, 4096 // S + 4
        g = torch.Generator(device=dev)
        g.manual_seed(1)
        nb = P * HKV * S * D // 2
        kc = torch.randint(0, 256, (nb,), dtype=torch.uint8, device=dev, generator=g)
        vc = torch.randint(0, 256, (nb,), dtype=torch.uint8, device=dev, generator=g)
        inv = float(np.float32(1.0) / np.sqrt(np.float32(D)))
        e = torch.randint(0, 3, (2 * P * HKV * S,), device=dev, generator=g)
        sc = (torch.ldexp(torch.ones_like(e, dtype=torch.float32), e - 2) * inv).contiguous()
        signs = torch.ones(D, device=dev)
        q = torch.randn((1, HQ, D), device=dev, generator=g).bfloat16()
        tab = torch.randperm(P, device=dev, generator=g)[: ctx_len // S].int().reshape(1, -1).contiguous()
        lens = torch.tensor([ctx_len], dtype=torch.int32, device=dev)
        out = torch.zeros((1, HQ, D), dtype=torch.bfloat16, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        res = {"profile": "config3", "kv_bytes": ctx_len * HKV * (D + 8), "us_per_decode": {}}
        for splits in (1, 2, 4, 8, 16, 0):
            n = splits if splits else tq.choose_splits(1, HKV, S, ctx_len)
            ws = torch.zeros(tq.decode_workspace_floats(1, HQ, HKV, D, n), device=dev)

            def call():
                tq.decode_splitk(q, kc, vc, sc, tab, lens, signs, out, num_heads=HQ, num_kv_heads=HKV,
                                 head_size=D, block_size=S, num_blocks=P, inv_sqrt_len=inv,
                                 softmax_scale=inv, splits=splits, max_context_hint=ctx_len, workspace=ws,
                                 output_stage=1)
            for _ in range(5):
                call()
            ts = []
            for _ in range(20):
                flush.fill_(1)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                call()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b) * 1e3)
            res["us_per_decode"]["auto(%d)" % n if splits == 0 else str(splits)] = round(statistics.median(ts), 1)
        print(json.dumps(res))
    elif args.profile == "lm_decode":
        rng = np.random.default_rng(0)
        ctx = rng.integers(2048, 4097, size=BATCH)
        pages = (ctx + S - 1) // S
        P = int(pages.sum()) + 8
        tables = np.zeros((BATCH, int(pages.max())), np.int32)
        perm, at = rng.permutation(P), 0
        for b in range(BATCH):
            tables[b, :pages[b]] = perm[at:at + pages[b]]
            at += int(pages[b])
        g = torch.Generator(device=dev)
        g.manual_seed(1)
        nb = P * HKV * S * D // 2
        kc = torch.randint(0, 256, (nb,), dtype=torch.uint8, device=dev, generator=g)
        vc = torch.randint(0, 256, (nb,), dtype=torch.uint8, device=dev, generator=g)
        sc = (torch.rand(2 * P * HKV * S, device=dev, generator=g) * 0.05 + 0.05).contiguous()
        q = torch.randn((BATCH, HQ, D), device=dev, generator=g).bfloat16()
        splits = 2
        ws = torch.zeros(BATCH * HKV * splits * (HQ // HKV) * (16 + D), device=dev)
        out = torch.zeros((BATCH, HQ, D), device=dev)
        dt, dc = torch.from_numpy(tables).to(dev), torch.from_numpy(ctx.astype(np.int32)).to(dev)
        for _ in range(5):
            tq.decode_lloydmax(q, kc, vc, sc, dt, dc, out, ws, num_heads=HQ, num_kv_heads=HKV,
                               head_size=D, block_size=S, num_blocks=P, splits=splits,
                               softmax_scale=float(1.0 / np.sqrt(D)), output_stage=1)
        torch.cuda.synchronize()
        print(json.dumps({"profile": "lm_decode", "kv_bytes": kv_bytes(ctx), "splits": splits}))
    elif args.profile == "scatter":
        w = build_workload(torch, dev, 11, context_lengths(11, BATCH, 2048, 4096))
        dk, dv, dslots = w["hk"].to(dev), w["hv"].to(dev), w["hslots"].to(dev)
        for _ in range(5):
            tq.reshape_scatter(dk, dv, w["key_cache"], w["value_cache"], w["scale_cache"], dslots,
                               w["signs"], None, num_requests=BATCH, num_kv_heads=HKV, head_size=D,
                               block_size=S, num_blocks=w["total_pages"], inv_sqrt_len=w["inv"])
        torch.cuda.synchronize()
        print(json.dumps({"profile": "scatter", "tokens": BATCH}))
    elif args.profile == "nz_import":
        P, H, SS = 2048, 4, 128
        g = torch.Generator(device=dev)
        g.manual_seed(3)
        nzk = torch.randint(0, 256, (P * SS * H * 128,), dtype=torch.uint8, device=dev, generator=g)
        nzv = torch.randint(0, 256, (P * SS * H * 128,), dtype=torch.uint8, device=dev, generator=g)
        nzs = torch.rand(P * SS * 8, device=dev, generator=g) + 0.5
        kc, vc = torch.empty_like(nzk), torch.empty_like(nzv)
        sc = torch.empty(2 * P * H * SS, dtype=torch.float32, device=dev)
        for _ in range(5):
            tq.nz_kv4_import(nzk, nzv, nzs, kc, vc, sc, num_kv_heads=H, block_size=SS, num_blocks=P)
        torch.cuda.synchronize()
        print(json.dumps({"profile": "nz_import",
                          "bytes": 2 * (2 * nzk.numel()) + P * SS * 8 * 4 + 2 * P * H * SS * 4}))
    elif args.profile in ("decode", "decode_d256"):
        if args.profile == "decode_d256":
            # the reference kernels' own geometry: head size 256, 16 query / 4 KV heads
            _use_reference_geometry()
        ctx = context_lengths(11, BATCH, 2048, 4096)
        w = build_workload(torch, dev, 11, ctx)
        splits = tq.choose_splits(BATCH, HKV, S, int(w["ctx"].max()),
                                  torch.cuda.get_device_properties(dev).multi_processor_count)
        ws = torch.zeros(tq.decode_workspace_floats(BATCH, HQ, HKV, D, splits), dtype=torch.float32,
                         device=dev)
        dq, dctx = w["hq"].to(dev), w["hctx"].to(dev)
        for _ in range(5):
            tq.decode_splitk_export(dq, w["key_cache"], w["value_cache"], w["scale_cache"],
                                    w["tables"], dctx, w["signs"], ws, num_heads=HQ,
                                    num_kv_heads=HKV, head_size=D, block_size=S,
                                    num_blocks=w["total_pages"], inv_sqrt_len=w["inv"],
                                    splits=0, softmax_scale=float(1.0 / np.sqrt(D)),
                                    max_context_hint=int(w["ctx"].max()))
        torch.cuda.synchronize()
        print(json.dumps({"profile": args.profile, "kv_bytes": kv_bytes(w["ctx"]), "splits": int(splits)}))
    else:
        T, H = 65536, 8
        g = torch.Generator(device=dev)
        g.manual_seed(2)
        lm = args.profile == "lm_reshape"
        if args.profile == "reshape_a8":
            k = torch.randint(-127, 128, (T, H * D), device=dev, generator=g, dtype=torch.int8)
            v = torch.randint(-127, 128, (T, H * D), device=dev, generator=g, dtype=torch.int8)
        else:
            k = torch.randn((T, H * D), device=dev, generator=g).bfloat16()
            v = torch.randn((T, H * D), device=dev, generator=g).bfloat16()
        P = T // S
        kc = torch.empty(P * H * S * D // 2, dtype=torch.uint8, device=dev)
        vc = torch.empty_like(kc)
        sc = torch.empty(2 * P * H * S, dtype=torch.float32, device=dev)
        perm = torch.randperm(P, device=dev, generator=g)
        slots = (perm[:, None] * S + torch.arange(S, device=dev)[None, :]).reshape(-1).int().contiguous()
        signs = torch.ones(D, device=dev)
        for _ in range(5):
            if lm:
                tq.reshape_and_cache_lloydmax(k, v, kc, vc, sc, slots, num_kv_heads=H, head_size=D,
                                              block_size=S, num_blocks=P, inv_sqrt_len=0.0883883)
            else:
                tq.reshape_and_cache(k, v, kc, vc, sc, slots, signs, num_kv_heads=H, head_size=D,
                                     block_size=S, num_blocks=P, inv_sqrt_len=0.0883883)
        torch.cuda.synchronize()
        print(json.dumps({"profile": args.profile,
                          "bytes": 2 * T * H * D * k.element_size() + T * H * D + 2 * T * H * 4}))


def cpu_baseline_decode(w, args, sample=BATCH):
    """The FP64 CPU oracle on a bounded sample of the same workload, all host threads."""
    from oracle.bindings import Oracle
    o = Oracle()
    threads = max(1, o.hardware_threads())
    ctx = w["ctx"][:sample]
    kc, vc = w["key_cache"].cpu().numpy(), w["value_cache"].cpu().numpy()
    sc = w["scale_cache"].cpu().numpy()
    q = w["hq"][:sample].view(__import__("torch").int16).numpy().view(np.uint16)
    signs = w["signs"].cpu().numpy()
    t0 = time.perf_counter()
    o.decode(q, kc, vc, sc, w["tables_np"][:sample], ctx.astype(np.int32), signs, HQ, HKV, D, S,
             w["total_pages"], w["inv"], float(1.0 / np.sqrt(D)), 1, None, threads=threads)
    dt = time.perf_counter() - t0
    return {"value": round(kv_bytes(ctx) / dt / 1e9, 4), "unit": "GB/s", "cores": threads,
            "kind": "port", "seconds": round(dt, 2),
            "sample": f"decode of the first {sample} of {len(w['ctx'])} sequences "
                      f"({int(ctx.sum())} context tokens), FP64 oracle, {threads} threads"}


# ------------------------------------------------------------ reference arm
def run_reference(args):
    """The reference's CPU implementation of the path (its FP64 decode model, restated in
    oracle/tq_oracle.cpp) on the host cores, same metric, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from oracle.bindings import Oracle
    o = Oracle()
    threads = max(1, o.hardware_threads())
    long_ctx = args.workload == "long"
    sample = 2 if long_ctx else 4
    ctx = (np.full(sample, LONG_CTX, np.int64) if long_ctx else context_lengths(4, BATCH)[:sample]) + 1
    rng = np.random.default_rng(5)
    pages = (ctx + S - 1) // S
    P = int(pages.sum())
    tables = np.zeros((sample, int(pages.max())), np.int32)
    perm, at = rng.permutation(P), 0
    for b in range(sample):
        tables[b, :pages[b]] = perm[at:at + pages[b]]
        at += int(pages[b])
    kc = rng.integers(0, 256, P * HKV * S * D // 2, dtype=np.uint8)
    vc = rng.integers(0, 256, P * HKV * S * D // 2, dtype=np.uint8)
    inv = float(np.float32(1.0) / np.sqrt(np.float32(D)))
    sc = (np.ldexp(1.0, rng.integers(0, 3, 2 * P * HKV * S) - 2) * inv).astype(np.float32)
    from oracle.bindings import bf16_from_f32
    q = bf16_from_f32(rng.standard_normal((sample, HQ, D)).astype(np.float32))
    signs = np.where(rng.random(D) < 0.5, -1.0, 1.0).astype(np.float32)

    def step():
        o.decode(q, kc, vc, sc, tables, ctx.astype(np.int32), signs, HQ, HKV, D, S, P, inv,
                 float(1.0 / np.sqrt(D)), 1, None, threads=threads)
    for _ in range(min(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = kv_bytes(ctx) / dt / 1e9
    sample_txt = (f"decode of {sample} sequences of the workload ({int(ctx.sum())} context tokens) "
                  f"per step, FP64 CPU model, {threads} threads")
    print(json.dumps({
        "impl": "reference", "metric": "splitk_4bit_decode_kv_hbm_gbs", "value": round(value, 4),
        "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": min(args.warmup, 1),
        "ms_per_step": round(dt * 1e3, 2), "higher_is_better": True,
        "scaling": "strong" if long_ctx else "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": LONG_WORKLOAD if long_ctx else WORKLOAD, "sample": sample_txt},
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": sample_txt},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="ragged", choices=["ragged", "long"],
                    help="ragged: 64 sequences of 512..32768 tokens per GPU (the headline, weak scaling); "
                         "long: 128 sequences of 65536 tokens in the whole job (strong scaling)")
    ap.add_argument("--profile", default=None, choices=["decode", "decode_d256", "config3", "reshape", "reshape_a8", "lm_decode", "lm_reshape", "scatter", "nz_import"],
                    help="run a small case of one kernel (for ncu), print no bench line")
    args = ap.parse_args()
    if args.profile:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
