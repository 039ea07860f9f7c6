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
over ranks. Every output that is timed is checked against the CPU oracle first; a
failed check ends the run with a non-zero exit code. `extra` carries the rest of the
metric: reshape tokens/s for int8 and bf16 activations at both head sizes, decode at
head size 256, microseconds per decode at batch 1 / context 4096 per split count, the
long-context configuration's share at this GPU count, the in-place NZ-tiled decode.
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
# The CPU arms time this many sequences of the ragged batch per step (the first ones of seed 4).
CPU_SAMPLE = 8
ABS_TOL, REL_TOL = 1e-3, 2e-3     # decode output vs the FP64 oracle


def kv_bytes(ctx_lens, hkv=None, d=None) -> int:
    from ascend_micro_harness_b200.sharding import kv_bytes as _kv
    return _kv(ctx_lens, HKV if hkv is None else hkv, D if d is None else d)


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


def summary(samples_ms):
    """min / mean / p50 / p95 / p99 of per-call device-event samples, in microseconds (the
    reference's benchmark protocol)."""
    s = sorted(samples_ms)
    pick = lambda q: s[min(len(s) - 1, max(0, int(np.ceil(q * len(s))) - 1))]
    return {"min_us": round(s[0] * 1e3, 2), "mean_us": round(statistics.fmean(s) * 1e3, 2),
            "p50_us": round(statistics.median(s) * 1e3, 2), "p95_us": round(pick(0.95) * 1e3, 2),
            "p99_us": round(pick(0.99) * 1e3, 2), "samples": len(s)}


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


def fail(msg):
    print(f"bench.py: verification failed: {msg}", file=sys.stderr)
    sys.exit(3)


# ----------------------------------------------------------------- our arm
def build_workload(torch, dev, seed, ctx=None, hq=None, hkv=None, d=None):
    """Seeded synthetic paged cache in HBM, generated directly in quantised form."""
    hq, hkv, d = hq or HQ, hkv or HKV, d or D
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
    nbytes = total_pages * hkv * S * d // 2
    key_cache = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=dev, generator=g)
    value_cache = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=dev, generator=g)
    inv = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    e = torch.randint(0, 3, (2 * total_pages * hkv * S,), device=dev, generator=g)
    scale_cache = (torch.ldexp(torch.ones_like(e, dtype=torch.float32), e - 2) * inv).contiguous()
    signs = torch.where(torch.rand(d, device=dev, generator=g) < 0.5, -1.0, 1.0).float()
    # per-step host inputs (pinned): one new token per sequence, the query, slots, lengths
    hk = torch.randn((B, hkv * d), generator=torch.Generator().manual_seed(seed)).bfloat16().pin_memory()
    hv = torch.randn((B, hkv * d), generator=torch.Generator().manual_seed(seed + 2)).bfloat16().pin_memory()
    hq_t = torch.randn((B, hq, d), generator=torch.Generator().manual_seed(seed + 3)).bfloat16().pin_memory()
    slots = np.array([tables[b, ctx[b] // S] * S + ctx[b] % S for b in range(B)], np.int32)
    hslots = torch.from_numpy(slots).pin_memory()
    hctx = torch.from_numpy((ctx + 1).astype(np.int32)).pin_memory()
    return dict(ctx=ctx + 1, total_pages=total_pages, max_blocks=max_blocks, inv=inv,
                key_cache=key_cache, value_cache=value_cache, scale_cache=scale_cache, signs=signs,
                tables=torch.from_numpy(tables).to(dev), hk=hk, hv=hv, hq=hq_t, hslots=hslots,
                hctx=hctx, tables_np=tables, hq_heads=hq, hkv_heads=hkv, d=d)


def bits16(t):
    import torch
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def verify_step(torch, tq, w, before, out, nseq, sample=3):
    """The step that is about to be timed, checked: the scatter's cache image against the
    oracle's scatter writer (every byte and scale bit of the whole pool), and the decode output
    of `sample` sequences (the longest, the shortest and one in between) against the FP64
    oracle over that cache."""
    from oracle.bindings import Oracle
    o = Oracle()
    hq, hkv, d = w["hq_heads"], w["hkv_heads"], w["d"]
    kc0, vc0, sc0 = before
    signs = w["signs"].cpu().numpy()
    ekc, evc, esc = kc0.copy(), vc0.copy(), sc0.copy()
    o.reshape_scatter(bits16(w["hk"]), bits16(w["hv"]), w["hslots"].numpy(), signs, None, nseq, hkv, d, S,
                      w["total_pages"], w["inv"], ekc, evc, esc)
    kc1, vc1, sc1 = (w[k].cpu().numpy() for k in ("key_cache", "value_cache", "scale_cache"))
    if not (np.array_equal(kc1, ekc) and np.array_equal(vc1, evc)
            and np.array_equal(sc1.view(np.uint32), esc.view(np.uint32))):
        fail("the scatter writer's cache image differs from the oracle's")
    order = np.argsort(w["ctx"])
    pick = sorted({int(order[0]), int(order[len(order) // 2]), int(order[-1])})[:sample]
    q = bits16(w["hq"])[pick]
    want = o.decode(q, kc1, vc1, sc1, w["tables_np"][pick], w["ctx"][pick].astype(np.int32), signs, hq, hkv, d, S,
                    w["total_pages"], w["inv"], float(1.0 / np.sqrt(d)), 1, None, threads=max(1, o.hardware_threads()))
    got = out.float().cpu().numpy()[pick]
    err = np.abs(got - want)
    bound = ABS_TOL + REL_TOL * np.abs(want) + 2.0 ** -8 * np.abs(want)   # + half an ulp of the bf16 output
    if not np.isfinite(got).all() or (err > bound).any():
        fail(f"decode output off by {(err / bound).max():.2f}x the tolerance on sequences {pick}")
    return {"scatter": "bit-exact (whole pool)", "decode_sequences": pick,
            "decode_worst_over_tolerance": round(float((err / bound).max()), 3)}


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
    warmup = max(args.warmup, 3)
    res = fused_step_bench(torch, tq, dev, dist, ctx_all[np.asarray(mine)], 4 + rank, args.steps, warmup,
                           verify=not args.no_verify, e2e=True, sampler=ClockSampler(local) if rank == 0 else None)
    clocks = res["clocks"]
    _, total_bytes = aggregate(0.0, res["bytes"], dist, dev)

    # the long-context configuration's share at this GPU count, on every rank (strong scaling)
    extra = {}
    if not long_ctx and not args.no_extra and LONG_BATCH % world == 0:
        share = partition_sequences(np.full(LONG_BATCH, LONG_CTX, np.int64), world, "round_robin")[rank]
        lres = fused_step_bench(torch, tq, dev, dist, np.full(len(share), LONG_CTX, np.int64), 40 + rank,
                                max(5, min(args.steps, 10)), 3, verify=False, e2e=False,
                                sampler=ClockSampler(local) if rank == 0 else None)
        _, long_total = aggregate(0.0, lres["bytes"], dist, dev)
        if rank == 0:
            peak, _ = measured_peak_gbs()
            extra["long_context"] = {
                "workload": LONG_WORKLOAD, "scaling": "strong", "sequences_per_gpu": len(share),
                "ms_per_step": round(lres["ms_step"], 4),
                "kv_gbs_all_gpus": round(long_total / (lres["ms_step"] * 1e-3) / 1e9, 1),
                "decode_kernel_us_rank0": round(lres["kernel_ms"] * 1e3, 1),
                "decode_kernel_frac_of_hbm_peak_rank0": round(lres["bytes"] / (lres["kernel_ms"] * 1e-3) / 1e9 / peak, 4),
                "clocks": lres["clocks"]}
        if world == 1:
            # what one GPU of eight would be handed (16 of the 128 sequences), timed on this GPU: the
            # ratio of the two step times is the strong-scaling factor an 8-GPU run can reach at best,
            # since the path has no exchange step
            eighth = LONG_BATCH // 8
            # The full job above runs into the board's power cap (its record says so); a GPU of eight
            # would start its share from idle, so this one rests first. Measured straight after the
            # full job the share reads 0.24-0.26 ms instead of 0.215.
            time.sleep(0.5)
            sres = fused_step_bench(torch, tq, dev, dist, np.full(eighth, LONG_CTX, np.int64), 48,
                                    max(5, min(args.steps, 10)), 3, verify=False, e2e=False,
                                    sampler=ClockSampler(local))
            extra["long_context"]["one_eighth_share"] = {
                "sequences": eighth, "ms_per_step": round(sres["ms_step"], 4),
                "decode_kernel_us": round(sres["kernel_ms"] * 1e3, 1),
                "decode_kernel_frac_of_hbm_peak": round(sres["bytes"] / (sres["kernel_ms"] * 1e-3) / 1e9 / peak, 4),
                "step_time_ratio_full_over_share": round(lres["ms_step"] / sres["ms_step"], 2),
                "clocks": sres["clocks"]}

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        ms_step = res["ms_step"]
        value = total_bytes / (ms_step * 1e-3) / 1e9
        achieved = res["bytes"] / (res["kernel_ms"] * 1e-3) / 1e9
        if not args.no_extra:
            extra.update(side_measurements(torch, tq, dev, args))
        nseq = len(mine)
        line = {
            "metric": "splitk_4bit_decode_kv_hbm_gbs", "value": round(value, 1), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "strong" if long_ctx else "weak",
            "vs_baseline": None, "dtype": "int4 codes; QK s8 x s8 -> s32, PV f16 x f16 -> f32", "data": "synthetic",
            "config": {"workload": LONG_WORKLOAD if long_ctx else WORKLOAD, "batch_per_gpu": nseq, "q_heads": HQ,
                       "kv_heads": HKV, "head_dim": D, "page_tokens": S, "splits": res["splits"],
                       "kv_bytes_per_gpu": res["bytes"],
                       "l2": "inputs larger than L2 (%.2f GB of cache read per step)" % (res["bytes"] / 1e9),
                       "parallelism": f"{nseq * world} sequences dealt to {world} GPU(s) "
                                      + ("round robin" if long_ctx else "by total context (longest first)")
                                      + f", {nseq} each, no collective"},
            "verified": res["verified"],
            "step_us": res["step_stats"],
            "decode_us_per_step": round(res["kernel_ms"] * 1e3, 1),
            "decode_kernel_us": res["kernel_stats"],
            "step_minus_decode_us": round((ms_step - res["kernel_ms"]) * 1e3, 1),
            "e2e": {"value": round(total_bytes / (res["ms_e2e"] * 1e-3) / 1e9, 1),
                    "unit": "GB/s", "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"],
                    "ms_per_step": round(res["ms_e2e"], 4), "issue": res["e2e_issue"]},
            "gpu_launches": 3 * args.steps,
            "issue": res["issue"],
            "roofline": {"kernel": "tq_decode_partial_kernel<128>", "bound": "hbm",
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}",
                         "traffic": int(res["bytes"] * DECODE_TRAFFIC_BYTES_PER_ALGORITHMIC_BYTE)},
            "clocks": clocks,
            "extra": extra,
        }
        if world == 1:
            line["cpu_baseline"] = cpu_baseline_decode(None, 2 if long_ctx else CPU_SAMPLE, long_ctx,
                                                       steps=3, warmup=1)
            if not args.no_extra:
                line["cpu_baseline"]["reshape"] = cpu_baseline_reshape()
        print(json.dumps(line))
        if args.csv:
            # the samples behind step_us / decode_kernel_us, one row per timed step (the reference's
            # benchmarks write the same kind of file)
            with open(args.csv, "w") as f:
                f.write("sample,step_us,decode_kernel_us\n")
                ks = res["kernel_samples_ms"]
                for i, t in enumerate(res["step_samples_ms"]):
                    k = f"{ks[i] * 1e3:.3f}" if i < len(ks) else ""
                    f.write(f"{i},{t * 1e3:.3f},{k}\n")
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# dram bytes (read + write) per algorithmic byte of the decode kernel, from an ncu capture of a
# small ragged case: dram__bytes_read.sum + dram__bytes_write.sum over the case's KV bytes.
# Traffic grows with the cache bytes read, so the full launch is scaled by its algorithmic bytes.
DECODE_TRAFFIC_BYTES_PER_ALGORITHMIC_BYTE = 1.0321


def fused_step_bench(torch, tq, dev, dist, ctx, seed, steps, warmup, verify, e2e, sampler=None):
    """Builds the paged cache for `ctx`, verifies one step against the oracle, then times
    `steps` fused steps (device-resident inputs), the same through host buffers, and the decode
    kernel on its own. Returns milliseconds (max over ranks where a group is given)."""
    from ascend_micro_harness_b200.sharding import aggregate
    w = build_workload(torch, dev, seed=seed, ctx=ctx)
    nseq = len(ctx)
    ctx1 = w["ctx"]
    splits = tq.choose_splits(nseq, HKV, S, int(ctx1.max()),
                              torch.cuda.get_device_properties(dev).multi_processor_count)
    ws = torch.empty(tq.decode_workspace_floats(nseq, HQ, HKV, D, splits), dtype=torch.float32, device=dev)
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

    def decode():
        tq.decode_splitk(dq, w["key_cache"], w["value_cache"], w["scale_cache"], w["tables"], dctx, w["signs"],
                         out, num_heads=HQ, splits=0, softmax_scale=scale, max_context_hint=int(ctx1.max()),
                         workspace=ws, output_stage=tq.OUT_UNROTATED, status=status, **geom)

    # the two kernels of decode() launched one by one, for timing the dominant one alone
    def export():
        tq.decode_splitk_export(dq, w["key_cache"], w["value_cache"], w["scale_cache"], w["tables"], dctx,
                                w["signs"], ws, num_heads=HQ, splits=0, softmax_scale=scale,
                                max_context_hint=int(ctx1.max()), status=status, **geom)

    def combine():
        tq.splitk_combine(ws, w["signs"], None, out, items=nseq * HKV, rows=HQ // HKV, rows_stride=HQ // HKV,
                          head_size=D, splits=splits, output_stage=tq.OUT_UNROTATED, inv_sqrt_len=w["inv"])

    # the fused step as one call of the library: the decode is scheduled under the writer
    def step():
        tq.decode_step(dk, dv, dslots, dq, w["key_cache"], w["value_cache"], w["scale_cache"], w["tables"], dctx,
                       w["signs"], out, num_heads=HQ, splits=0, softmax_scale=scale,
                       max_context_hint=int(ctx1.max()), workspace=ws, output_stage=tq.OUT_UNROTATED,
                       status=status, **geom)

    def e2e_body():
        dev_in.copy_(host_in, non_blocking=True)
        step()
        hout.copy_(out, non_blocking=True)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- verify before the clock starts
    verified = False
    if verify:
        before = tuple(w[k].cpu().numpy() for k in ("key_cache", "value_cache", "scale_cache"))
        step()
        torch.cuda.synchronize()
        if int(status.item()) != 0:
            fail(f"device status word {int(status.item())}")
        verified = verify_step(torch, tq, w, before, out, nseq)
        del before

    def timed(fn, n):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(n):
            fn()
        ev1.record()
        barrier()
        ms, _ = aggregate(ev0.elapsed_time(ev1), 0, dist, dev)   # max over ranks
        return ms

    def sampled(fn, n):
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        torch.cuda.synchronize()
        for a, b in evs:
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]

    for _ in range(warmup):
        step()
    # The timed steps are issued as replays of one captured step (scatter, export, combine): one host call
    # per step, so a short run is not dominated by the first step's launch gaps.
    step_issue, issue = step, "3 launches per step"
    try:
        torch.cuda.synchronize()
        step_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(step_graph):
            step()
        step_issue, issue = step_graph.replay, "one CUDA graph replay (3 kernels) per step"
        step_issue()
    except Exception as exc:
        print(f"bench.py: CUDA graph capture of the step failed ({exc}); eager launches", file=sys.stderr)
        step_issue, issue = step, "3 launches per step"
    if sampler is not None:      # clocks and throttle reasons DURING the timed regions only
        sampler.start()
    ms_total = timed(step_issue, steps)
    step_samples = sampled(step_issue, steps)

    ms_e2e, e2e_issue = float("nan"), None
    if e2e:
        # The end-to-end step as a serving loop issues it: host->device copy of the step's inputs,
        # the three launches and the device->host copy of the output captured once as a CUDA graph
        # (the library neither allocates nor synchronises, so its launches are capturable), then
        # one graph launch and one stream synchronisation per step.
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
        except Exception as exc:                 # capture refused: issue the calls one by one
            print(f"bench.py: CUDA graph capture of the end-to-end step failed ({exc}); eager calls",
                  file=sys.stderr)
            e2e_graph = None

        def e2e_step():
            if e2e_graph is not None:
                e2e_graph.replay()
            else:
                e2e_body()
            torch.cuda.current_stream().synchronize()
        for _ in range(3):
            e2e_step()
        ms_e2e = timed(e2e_step, steps) / steps
        e2e_issue = ("one CUDA graph (copy in, 3 kernels, copy out) + stream sync per step"
                     if e2e_graph is not None else "5 calls + stream sync per step")

    # the dominant kernel on its own, CUDA events on the launching stream
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    barrier()
    step()   # one untimed step: the first launches after a barrier start on an idle GPU
    for a, b in evs:
        scatter()
        a.record()
        export()
        b.record()
        combine()
    barrier()
    kernel_samples = [a.elapsed_time(b) for a, b in evs]
    clocks = sampler.stop() if sampler is not None else None
    if int(status.item()) != 0:
        fail(f"device status word {int(status.item())}")
    return {"clocks": clocks, "ms_step": ms_total / steps, "ms_e2e": ms_e2e, "kernel_ms": statistics.median(kernel_samples),
            "step_stats": summary(step_samples), "kernel_stats": summary(kernel_samples),
            "step_samples_ms": list(step_samples), "kernel_samples_ms": list(kernel_samples),
            "bytes": kv_bytes(ctx1), "splits": int(splits), "verified": verified, "issue": issue,
            "e2e_issue": e2e_issue, "h2d": int(host_in.numel()), "d2h": int(hout.numel() * hout.element_size())}


def cold_samples(torch, fn, n, flush):
    """Per-call device-event samples with L2 evicted before every call (a write larger than L2)."""
    out = []
    for _ in range(n):
        flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return out


def reshape_case(torch, tq, dev, dtype, H, d, T, reps, verify=True):
    """reshape_and_cache on T tokens x H KV heads x d (permuted pages): verifies 256 sampled
    strips bit for bit against the oracle, then times back-to-back launches (inputs > L2)."""
    from oracle.bindings import Oracle
    g = torch.Generator(device=dev)
    g.manual_seed(2 + d + (1 if dtype == "int8" else 0))
    if dtype == "int8":
        k = torch.randint(-127, 128, (T, H * d), device=dev, generator=g, dtype=torch.int8)
        v = torch.randint(-127, 128, (T, H * d), device=dev, generator=g, dtype=torch.int8)
    else:
        # integer-valued bf16 (the bit-checkable form): N(0,1) x 16, clipped, rounded
        k = torch.clamp(torch.round(torch.randn((T, H * d), device=dev, generator=g) * 16), -127, 127).bfloat16()
        v = torch.clamp(torch.round(torch.randn((T, H * d), device=dev, generator=g) * 16), -127, 127).bfloat16()
    P = T // S
    kc = torch.empty(P * H * S * d // 2, dtype=torch.uint8, device=dev)
    vc = torch.empty_like(kc)
    sc = torch.empty(2 * P * H * S, dtype=torch.float32, device=dev)
    perm = torch.randperm(P, device=dev, generator=g)
    slots = (perm[:, None] * S + torch.arange(S, device=dev)[None, :]).reshape(-1).int().contiguous()
    signs = torch.where(torch.rand(d, device=dev, generator=g) < 0.5, -1.0, 1.0).float()
    inv = float(np.float32(1.0) / np.sqrt(np.float32(d)))

    def reshape():
        tq.reshape_and_cache(k, v, kc, vc, sc, slots, signs, num_kv_heads=H, head_size=d,
                             block_size=S, num_blocks=P, inv_sqrt_len=inv)
    reshape()
    torch.cuda.synchronize()
    if verify:
        o = Oracle()
        pick = np.sort(np.random.default_rng(d).choice(P, size=256, replace=False))
        rows = (torch.from_numpy(pick).to(dev)[:, None] * S + torch.arange(S, device=dev)[None, :]).reshape(-1)
        ks, vs = k[rows].cpu(), v[rows].cpu()
        ks = ks.numpy() if dtype == "int8" else bits16(ks)
        vs = vs.numpy() if dtype == "int8" else bits16(vs)
        ekc, evc, esc, _, bad = o.reshape_and_cache(ks, vs, np.arange(256 * S, dtype=np.int32),
                                                    np.where(signs.cpu().numpy() < 0, -1, 1).astype(np.int32), H, d,
                                                    S, 256, inv, threads=max(1, o.hardware_threads()))
        pages = perm[torch.from_numpy(pick).to(dev)].cpu().numpy()
        blk = H * S * d // 2
        gk = kc.view(P, blk)[torch.from_numpy(pages).to(dev)].cpu().numpy().reshape(-1)
        gv = vc.view(P, blk)[torch.from_numpy(pages).to(dev)].cpu().numpy().reshape(-1)
        gs = sc.view(2, P, H * S)[:, torch.from_numpy(pages).to(dev)].cpu().numpy().reshape(-1)
        if bad != -1 or not (np.array_equal(gk, ekc) and np.array_equal(gv, evc)
                             and np.array_equal(gs.view(np.uint32), esc.view(np.uint32))):
            fail(f"reshape_and_cache {dtype} d={d}: sampled strips differ from the oracle")
    for _ in range(3):
        reshape()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    torch.cuda.synchronize()
    for a, b in evs:
        a.record()
        reshape()
        b.record()
    torch.cuda.synchronize()
    samples = [a.elapsed_time(b) for a, b in evs]
    ms = statistics.median(samples)
    nbytes = 2 * T * H * d * k.element_size() + 2 * T * H * d // 2 + 2 * T * H * 4
    peak, _ = measured_peak_gbs()
    return {"workload": f"{dtype} prefill {T} tokens x {H} KV heads x {d}, permuted pages", "verified": bool(verify),
            "tokens_per_s": round(T / (ms * 1e-3)), "ms": round(ms, 4), "bytes": nbytes,
            "gbs": round(nbytes / (ms * 1e-3) / 1e9, 1),
            "frac_of_hbm_peak": round(nbytes / (ms * 1e-3) / 1e9 / peak, 4), "us": summary(samples)}


def decode_case(torch, tq, dev, hq, hkv, d, ctx, reps, seed=21):
    """The decode kernel alone on a seeded batch at another geometry (verified on 2 sequences)."""
    from oracle.bindings import Oracle
    w = build_workload(torch, dev, seed, ctx, hq=hq, hkv=hkv, d=d)
    B = len(ctx)
    dq, dctx = w["hq"].to(dev), w["hctx"].to(dev)
    n = tq.choose_splits(B, hkv, S, int(w["ctx"].max()), torch.cuda.get_device_properties(dev).multi_processor_count)
    ws = torch.empty(tq.decode_workspace_floats(B, hq, hkv, d, n), dtype=torch.float32, device=dev)
    out = torch.zeros((B, hq, d), dtype=torch.bfloat16, device=dev)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    scale = float(1.0 / np.sqrt(d))

    def decode():
        tq.decode_splitk(dq, w["key_cache"], w["value_cache"], w["scale_cache"], w["tables"], dctx, w["signs"], out,
                         num_heads=hq, num_kv_heads=hkv, head_size=d, block_size=S, num_blocks=w["total_pages"],
                         inv_sqrt_len=w["inv"], splits=0, softmax_scale=scale, max_context_hint=int(w["ctx"].max()),
                         workspace=ws, output_stage=tq.OUT_UNROTATED, status=st)
    decode()
    torch.cuda.synchronize()
    o = Oracle()
    pick = [int(np.argmin(w["ctx"])), int(np.argmax(w["ctx"]))]
    want = o.decode(bits16(w["hq"])[pick], w["key_cache"].cpu().numpy(), w["value_cache"].cpu().numpy(),
                    w["scale_cache"].cpu().numpy(), w["tables_np"][pick], w["ctx"][pick].astype(np.int32),
                    w["signs"].cpu().numpy(), hq, hkv, d, S, w["total_pages"], w["inv"], scale, 1, None,
                    threads=max(1, o.hardware_threads()))
    got = out.float().cpu().numpy()[pick]
    bound = ABS_TOL + (REL_TOL + 2.0 ** -8) * np.abs(want)
    if int(st.item()) != 0 or (np.abs(got - want) > bound).any():
        fail(f"decode at head size {d}: output outside the tolerance")
    for _ in range(3):
        decode()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    torch.cuda.synchronize()
    for a, b in evs:
        a.record()
        decode()
        b.record()
    torch.cuda.synchronize()
    samples = [a.elapsed_time(b) for a, b in evs]
    ms = statistics.median(samples)
    nbytes = kv_bytes(w["ctx"], hkv, d)
    peak, _ = measured_peak_gbs()
    return {"workload": f"{B} sequences of {int(ctx.min())}..{int(ctx.max())} tokens, {hq} q / {hkv} KV heads x {d}",
            "verified": True, "kv_bytes": nbytes, "ms": round(ms, 4), "gbs": round(nbytes / (ms * 1e-3) / 1e9, 1),
            "frac_of_hbm_peak": round(nbytes / (ms * 1e-3) / 1e9 / peak, 4), "us": summary(samples)}


def config3_case(torch, tq, dev):
    """Batch 1, 32 q / 8 KV heads, context 4096, shuffled table: microseconds per decode for
    explicit split counts and for the library's own choice, L2 evicted before every call."""
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
    res = {"workload": "batch 1, 32 q / 8 KV heads x 128, context 4096, L2 evicted before every call",
           "kv_bytes": ctx_len * HKV * (D + 8), "us_per_decode": {}, "warm_us_per_decode": {}}
    # what the same bracket reads around nothing and around a 32-element elementwise kernel:
    # the part of every figure below that is the method's, not the decode's
    tiny = torch.zeros(32, device=dev)
    res["floor_us"] = {"empty_bracket": summary(cold_samples(torch, lambda: None, 30, flush))["p50_us"],
                       "tiny_kernel": summary(cold_samples(torch, lambda: tiny.add_(1), 30, flush))["p50_us"]}
    for splits in (1, 2, 4, 8, 16, 32, 0):
        n = splits if splits else tq.choose_splits(1, HKV, S, ctx_len)
        ws = torch.zeros(tq.decode_workspace_floats(1, HQ, HKV, D, n), device=dev)

        def call():
            tq.decode_splitk(q, kc, vc, sc, tab, lens, signs, out, num_heads=HQ, num_kv_heads=HKV,
                             head_size=D, block_size=S, num_blocks=P, inv_sqrt_len=inv,
                             softmax_scale=inv, splits=splits, max_context_hint=ctx_len, workspace=ws,
                             output_stage=1)
        for _ in range(5):
            call()
        name = "auto" if splits == 0 else str(splits)
        res["us_per_decode"][name] = summary(cold_samples(torch, call, 30, flush))["p50_us"]
        warm = []
        for _ in range(30):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            call()
            b.record()
            torch.cuda.synchronize()
            warm.append(a.elapsed_time(b))
        res["warm_us_per_decode"][name] = summary(warm)["p50_us"]
    # the same decode as ONE launch: the persistent grid merges the records itself
    res["single_launch_us_per_decode"] = {}
    for slots in (8, 16, 32):
        ws = torch.zeros(tq.decode_workspace_floats(1, HQ, HKV, D, slots), device=dev)

        def one():
            tq.decode_splitk(q, kc, vc, sc, tab, lens, signs, out, num_heads=HQ, num_kv_heads=HKV,
                             head_size=D, block_size=S, num_blocks=P, inv_sqrt_len=inv,
                             softmax_scale=inv, splits=slots, max_context_hint=ctx_len, workspace=ws,
                             output_stage=1, persistent=True)
        for _ in range(5):
            one()
        res["single_launch_us_per_decode"][str(slots)] = summary(cold_samples(torch, one, 30, flush))["p50_us"]
    return res


def nz_case(torch, tq, dev, reps):
    """Decode over the fused decoder's NZ-tiled KV4 pools in place: 64 sequences of 2048..16384
    tokens, 16 q / 4 KV heads x 256, pages of 128 slots."""
    H, G, SS = 4, 4, 128
    rng = np.random.default_rng(17)
    ctx = rng.integers(2048, 16385, size=BATCH).astype(np.int64)
    pages = (ctx + SS - 1) // SS
    P = int(pages.sum()) + 8
    tables = np.zeros((BATCH, int(pages.max())), np.int32)
    perm, at = rng.permutation(P), 0
    for b in range(BATCH):
        tables[b, :pages[b]] = perm[at:at + pages[b]]
        at += int(pages[b])
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    nzk = torch.randint(0, 256, (P * SS * H * 128,), dtype=torch.uint8, device=dev, generator=g)
    nzv = torch.randint(0, 256, (P * SS * H * 128,), dtype=torch.uint8, device=dev, generator=g)
    nzs = (torch.rand(P * SS * 8, device=dev, generator=g) * 0.2 + 0.1).contiguous()
    q = torch.randn((BATCH, H * G, 256), device=dev, generator=g)
    dt, dc = torch.from_numpy(tables).to(dev), torch.from_numpy(ctx.astype(np.int32)).to(dev)
    n = tq.choose_splits(BATCH, H, SS, int(ctx.max()), torch.cuda.get_device_properties(dev).multi_processor_count)
    ws = torch.empty(tq.decode_workspace_floats(BATCH, H * G, H, 256, n), dtype=torch.float32, device=dev)
    out = torch.zeros((BATCH, H * G, 256), dtype=torch.float16, device=dev)
    st = torch.zeros(1, dtype=torch.int32, device=dev)

    def decode():
        tq.decode_splitk_nz(q, nzk, nzv, nzs, dt, dc, out, num_heads=H * G, num_kv_heads=H, block_size=SS,
                            num_blocks=P, softmax_scale=0.0625, splits=0, max_context_hint=int(ctx.max()),
                            workspace=ws, status=st)
    for _ in range(3):
        decode()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    torch.cuda.synchronize()
    for a, b in evs:
        a.record()
        decode()
        b.record()
    torch.cuda.synchronize()
    if int(st.item()) != 0:
        fail("in-place NZ decode: device status word set")
    samples = [a.elapsed_time(b) for a, b in evs]
    ms = statistics.median(samples)
    nbytes = int(ctx.sum()) * (H * 256 + 8 * 4)      # packed K + V rows and the 8-float scale record per slot
    peak, _ = measured_peak_gbs()
    return {"workload": "64 sequences of 2048..16384 tokens, 16 q / 4 KV heads x 256, NZ-tiled KV4 pools read in place",
            "kv_bytes": nbytes, "ms": round(ms, 4), "gbs": round(nbytes / (ms * 1e-3) / 1e9, 1),
            "frac_of_hbm_peak": round(nbytes / (ms * 1e-3) / 1e9 / peak, 4), "us": summary(samples)}


def persistent_case(torch, tq, dev, reps):
    """The single-launch persistent grid (tq_decode_splitk_persistent) on the ragged batch, beside
    the default two-kernel decode on the same inputs, with its worker census: segments per CTA
    and microseconds per segment boundary."""
    ctx = context_lengths(4)
    w = build_workload(torch, dev, 4, ctx)
    n = len(ctx)
    dq, dctx = w["hq"].to(dev), w["hctx"].to(dev)
    ws = torch.empty(tq.decode_workspace_floats(n, HQ, HKV, D, tq.MAX_SPLITS), dtype=torch.float32, device=dev)
    out = torch.zeros((n, HQ, D), dtype=torch.bfloat16, device=dev)
    ref = torch.zeros_like(out)
    geom = dict(num_heads=HQ, num_kv_heads=HKV, head_size=D, block_size=S, num_blocks=w["total_pages"],
                inv_sqrt_len=w["inv"], softmax_scale=float(1.0 / np.sqrt(D)), output_stage=tq.OUT_UNROTATED)
    args = (dq, w["key_cache"], w["value_cache"], w["scale_cache"], w["tables"], dctx, w["signs"])

    def persistent():
        tq.decode_splitk(*args, out, splits=0, workspace=ws, persistent=True, **geom)

    def default():
        tq.decode_splitk(*args, ref, splits=0, max_context_hint=int(w["ctx"].max()), workspace=ws, **geom)
    default()
    persistent()
    torch.cuda.synchronize()
    diff = (out.float() - ref.float()).abs().max().item()
    if not diff <= 2e-2:          # two bf16 roundings of results that agree to about 1e-3
        fail(f"persistent decode differs from the default decode by {diff}")

    def timed(fn):
        for _ in range(3):
            fn()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        torch.cuda.synchronize()
        for a, b in evs:
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return statistics.median(a.elapsed_time(b) for a, b in evs)
    ms_p, ms_d = timed(persistent), timed(default)
    cen = torch.zeros(10 * 1024, dtype=torch.int64, device=dev)
    tq.worker_census(cen)
    persistent()
    torch.cuda.synchronize()
    tq.worker_census(None)
    c = cen.cpu().numpy().reshape(-1, 10)
    c = c[c[:, 1] > 0]
    busy = (c[:, 1] - c[:, 0]) / 1e3
    nbytes = kv_bytes(w["ctx"])
    return {"workload": WORKLOAD + " (decode only)", "persistent_ms": round(ms_p, 4), "default_ms": round(ms_d, 4),
            "persistent_gbs": round(nbytes / (ms_p * 1e-3) / 1e9, 1), "default_gbs": round(nbytes / (ms_d * 1e-3) / 1e9, 1),
            "census": {"ctas": int(len(c)), "segments_per_cta": round(float(c[:, 3].mean()), 2),
                       "busy_us_mean": round(float(busy.mean()), 1), "busy_us_max": round(float(busy.max()), 1),
                       "tile_loop_us_mean": round(float(c[:, 2].mean() / 1e3), 1),
                       "boundary_us_per_segment": round(float(((busy - c[:, 2] / 1e3) / np.maximum(c[:, 3], 1)).mean()), 2)}}


def side_measurements(torch, tq, dev, args):
    """The rest of the metric on one GPU: reshape tokens/s (int8 and bf16, head sizes 128 and
    256; 1 GiB / 0.5 GiB of activations, far beyond L2), decode at the reference kernels' own
    geometry (4 KV heads x 256), microseconds per decode at batch 1 / context 4096 for split
    counts 1/2/4/8/16/auto, and the in-place decode of the fused decoder's cache."""
    reps = max(args.steps, 5)
    T = 262144
    cases = {
        "reshape_bf16": lambda: reshape_case(torch, tq, dev, "bf16", 8, 128, T, reps),
        "reshape_a8": lambda: reshape_case(torch, tq, dev, "int8", 8, 128, T, reps),
        "reshape_bf16_d256": lambda: reshape_case(torch, tq, dev, "bf16", 4, 256, T, reps),
        "reshape_a8_d256": lambda: reshape_case(torch, tq, dev, "int8", 4, 256, T, reps),
        "decode_d256": lambda: decode_case(torch, tq, dev, 16, 4, 256,
                                           context_lengths(9, BATCH, 2048, 16384), reps),
        "decode_config3_us": lambda: config3_case(torch, tq, dev),
        "decode_nz_inplace": lambda: nz_case(torch, tq, dev, reps),
        "decode_persistent": lambda: persistent_case(torch, tq, dev, reps),
    }
    only = [n for n in (args.side or "").split(",") if n]
    for n in only:
        if n not in cases:
            raise SystemExit(f"--side: unknown case {n!r}; known: {', '.join(cases)}")
    return {n: fn() for n, fn in cases.items() if not only or n in only}


def _use_reference_geometry():
    """Switch the module's workload constants to head size 256 with 16 query / 4 KV heads."""
    global D, HQ, HKV
    D, HQ, HKV = 256, 16, 4


def run_profile_case(args):
    """A small case of one kernel for an ncu capture: inputs larger than L2 but well under
    a GB on the device, a few warm-up launches and the captured ones.
      decode  : 64 sequences x 2048..4096 tokens (about 0.2 GB of cache): export of the per-split
                records (the dominant kernel) and the combine
      decode_persistent : the same batch on the single-launch persistent grid
      decode_d256 : the same at head size 256 with 16 query / 4 KV heads
      decode_nz   : the in-place decode of NZ-tiled pools, 64 sequences x 1024..2048 tokens
      config3 : batch 1, context 4096, split-K swept over 1/2/4/8/16/auto: prints microseconds per decode
      reshape : bf16 prefill of 65536 tokens x 8 KV heads x 128 (0.27 GB)
      reshape_a8 : the same prefill with int8 activations (0.13 GB)
      reshape_d256 / reshape_a8_d256 : the same at 4 KV heads x 256
      lm_decode  : the Lloyd-Max cache variant, 64 sequences x 2048..4096 tokens, 2 splits
      lm_reshape : its bf16 writer on the 65536-token prefill
      scatter    : the 1-token-per-sequence writer of a 64-sequence decode step
      nz_import  : the KV4/FP8 NZ-tiled importer, 2048 pages x 128 slots x 4 heads (0.27 GB in)"""
    import torch
    import ascend_micro_harness_b200 as tq
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if args.profile == "config3":
        print(json.dumps(dict(profile="config3", **config3_case(torch, tq, dev))))
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
    elif args.profile == "decode_nz":
        H, G, SS = 4, 4, 128
        rng = np.random.default_rng(17)
        ctx = rng.integers(1024, 2049, size=BATCH).astype(np.int64)
        pages = (ctx + SS - 1) // SS
        P = int(pages.sum()) + 8
        tables = np.zeros((BATCH, int(pages.max())), np.int32)
        perm, at = rng.permutation(P), 0
        for b in range(BATCH):
            tables[b, :pages[b]] = perm[at:at + pages[b]]
            at += int(pages[b])
        g = torch.Generator(device=dev)
        g.manual_seed(3)
        nzk = torch.randint(0, 256, (P * SS * H * 128,), dtype=torch.uint8, device=dev, generator=g)
        nzv = torch.randint(0, 256, (P * SS * H * 128,), dtype=torch.uint8, device=dev, generator=g)
        nzs = (torch.rand(P * SS * 8, device=dev, generator=g) * 0.2 + 0.1).contiguous()
        q = torch.randn((BATCH, H * G, 256), device=dev, generator=g)
        dt, dc = torch.from_numpy(tables).to(dev), torch.from_numpy(ctx.astype(np.int32)).to(dev)
        n = tq.choose_splits(BATCH, H, SS, int(ctx.max()))
        ws = torch.empty(tq.decode_workspace_floats(BATCH, H * G, H, 256, n), dtype=torch.float32, device=dev)
        out = torch.zeros((BATCH, H * G, 256), dtype=torch.float16, device=dev)
        for _ in range(5):
            tq.decode_splitk_nz(q, nzk, nzv, nzs, dt, dc, out, num_heads=H * G, num_kv_heads=H, block_size=SS,
                                num_blocks=P, softmax_scale=0.0625, splits=0, max_context_hint=int(ctx.max()),
                                workspace=ws)
        torch.cuda.synchronize()
        print(json.dumps({"profile": "decode_nz", "kv_bytes": int(ctx.sum()) * (H * 256 + 32)}))
    elif args.profile in ("decode", "decode_d256", "decode_persistent"):
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
        out = torch.zeros((BATCH, HQ, D), dtype=torch.bfloat16, device=dev)
        if args.profile == "decode_persistent":
            ws = torch.zeros(tq.decode_workspace_floats(BATCH, HQ, HKV, D, tq.MAX_SPLITS), dtype=torch.float32,
                             device=dev)
        for _ in range(5):
            if args.profile == "decode_persistent":
                tq.decode_splitk(dq, w["key_cache"], w["value_cache"], w["scale_cache"], w["tables"], dctx,
                                 w["signs"], out, num_heads=HQ, num_kv_heads=HKV, head_size=D, block_size=S,
                                 num_blocks=w["total_pages"], inv_sqrt_len=w["inv"], splits=0,
                                 softmax_scale=float(1.0 / np.sqrt(D)), workspace=ws, output_stage=1, persistent=True)
                continue
            tq.decode_splitk(dq, w["key_cache"], w["value_cache"], w["scale_cache"], w["tables"], dctx,
                             w["signs"], out, num_heads=HQ, num_kv_heads=HKV, head_size=D, block_size=S,
                             num_blocks=w["total_pages"], inv_sqrt_len=w["inv"], splits=0,
                             softmax_scale=float(1.0 / np.sqrt(D)), max_context_hint=int(w["ctx"].max()),
                             workspace=ws, output_stage=1)
        torch.cuda.synchronize()
        print(json.dumps({"profile": args.profile, "kv_bytes": kv_bytes(w["ctx"]), "splits": int(splits)}))
    else:
        T = 65536
        H, d = (4, 256) if args.profile.endswith("d256") else (8, 128)
        g = torch.Generator(device=dev)
        g.manual_seed(2)
        lm = args.profile == "lm_reshape"
        if args.profile.startswith("reshape_a8"):
            k = torch.randint(-127, 128, (T, H * d), device=dev, generator=g, dtype=torch.int8)
            v = torch.randint(-127, 128, (T, H * d), device=dev, generator=g, dtype=torch.int8)
        else:
            k = torch.randn((T, H * d), device=dev, generator=g).bfloat16()
            v = torch.randn((T, H * d), device=dev, generator=g).bfloat16()
        P = T // S
        kc = torch.empty(P * H * S * d // 2, dtype=torch.uint8, device=dev)
        vc = torch.empty_like(kc)
        sc = torch.empty(2 * P * H * S, dtype=torch.float32, device=dev)
        perm = torch.randperm(P, device=dev, generator=g)
        slots = (perm[:, None] * S + torch.arange(S, device=dev)[None, :]).reshape(-1).int().contiguous()
        signs = torch.ones(d, device=dev)
        for _ in range(5):
            if lm:
                tq.reshape_and_cache_lloydmax(k, v, kc, vc, sc, slots, num_kv_heads=H, head_size=d,
                                              block_size=S, num_blocks=P, inv_sqrt_len=0.0883883)
            else:
                tq.reshape_and_cache(k, v, kc, vc, sc, slots, signs, num_kv_heads=H, head_size=d,
                                     block_size=S, num_blocks=P, inv_sqrt_len=0.0883883)
        torch.cuda.synchronize()
        print(json.dumps({"profile": args.profile,
                          "bytes": 2 * T * H * d * k.element_size() + T * H * d + 2 * T * H * 4}))


# ------------------------------------------------------------ CPU arms
def cpu_decode_sample(sample, long_ctx):
    """The first `sample` sequences of the ragged batch (seed 4) as a self-contained host
    workload: context lengths, a paged cache in quantised form, block tables, queries."""
    from oracle.bindings import bf16_from_f32
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
    q = bf16_from_f32(rng.standard_normal((sample, HQ, D)).astype(np.float32))
    signs = np.where(rng.random(D) < 0.5, -1.0, 1.0).astype(np.float32)
    return dict(ctx=ctx, P=P, tables=tables, kc=kc, vc=vc, sc=sc, q=q, signs=signs, inv=inv)


def cpu_baseline_decode(_unused, sample, long_ctx, steps, warmup):
    """The FP64 CPU model of the decode (oracle/tq_oracle.cpp, a restatement: the reference's own
    decode model is bound to its fixture geometry) on a bounded sample, all host threads. The
    same function, sample and thread count serve `--impl reference`."""
    from oracle.bindings import Oracle
    o = Oracle()
    threads = max(1, o.hardware_threads())
    c = cpu_decode_sample(sample, long_ctx)

    def step():
        o.decode(c["q"], c["kc"], c["vc"], c["sc"], c["tables"], c["ctx"].astype(np.int32), c["signs"], HQ, HKV, D, S,
                 c["P"], c["inv"], float(1.0 / np.sqrt(D)), 1, None, threads=threads)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    nbytes = kv_bytes(c["ctx"])
    return {"value": round(nbytes / dt / 1e9, 4), "unit": "GB/s", "cores": threads, "kind": "port",
            "seconds_per_step": round(dt, 3),
            "sample": f"decode of the first {sample} sequences of the workload ({int(c['ctx'].sum())} context "
                      f"tokens) per step, FP64 CPU model, {threads} threads"}


def cpu_baseline_reshape(tokens=131072):
    """reshape_and_cache on the host: the reference's own tq_oracle::compute_oracle_reference
    (tests/common/turboquant_oracle.hpp:476-513) compiled from the reference checkout into
    oracle/_ref/libtq_ref.so, its strips spread over all host threads; the restated oracle where
    that library was not built. int8 activations, 8 KV heads x 128."""
    from oracle.bindings import Oracle, Reference
    o = Oracle()
    threads = max(1, o.hardware_threads())
    H, d = 8, 128
    rng = np.random.default_rng(6)
    k = rng.integers(-127, 128, (tokens, H * d), dtype=np.int64).astype(np.int8)
    v = rng.integers(-127, 128, (tokens, H * d), dtype=np.int64).astype(np.int8)
    P = tokens // S
    slots = (rng.permutation(P)[:, None] * S + np.arange(S)[None, :]).astype(np.int32).reshape(-1)
    if Reference.available():
        r = Reference()
        kind = "reference"
        run = lambda: r.writer_reference(k, v, slots, H, d, S, P, threads=threads)
    else:
        kind = "port"
        signs = o.writer_signs(d)
        run = lambda: o.reshape_and_cache(k, v, slots, signs, H, d, S, P, float(np.float32(1) / np.sqrt(np.float32(d))),
                                          threads=threads)
    t0 = time.perf_counter()
    run()
    dt = time.perf_counter() - t0
    return {"value": round(tokens / dt), "unit": "tokens/s", "cores": threads, "kind": kind, "seconds": round(dt, 2),
            "gbs": round(tokens * H * (3 * d + 8) / dt / 1e9, 4),
            "sample": f"{tokens} tokens x {H} KV heads x {d} int8 (half of the timed GPU case), {threads} threads"}


def run_reference(args):
    """The reference's CPU implementation of the path on the host cores, same metric, bounded
    sample per step: the FP64 decode model (restated in oracle/tq_oracle.cpp; the reference's own
    is bound to its fixture geometry) with the thread count, sample and warm-up count of the
    main arm's cpu_baseline; the reshape leg runs the reference's own writer model compiled from
    its sources (oracle/_ref/libtq_ref.so)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    long_ctx = args.workload == "long"
    warmup = max(args.warmup, 3)
    base = cpu_baseline_decode(None, 2 if long_ctx else CPU_SAMPLE, long_ctx, steps=args.steps, warmup=warmup)
    base["reshape"] = cpu_baseline_reshape()
    print(json.dumps({
        "impl": "reference", "metric": "splitk_4bit_decode_kv_hbm_gbs", "value": base["value"],
        "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(base["seconds_per_step"] * 1e3, 2), "higher_is_better": True,
        "scaling": "strong" if long_ctx else "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": LONG_WORKLOAD if long_ctx else WORKLOAD, "sample": base["sample"]},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
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
    ap.add_argument("--no-extra", action="store_true", help="skip the side measurements of `extra`")
    ap.add_argument("--no-verify", action="store_true", help="skip the oracle check before timing")
    ap.add_argument("--csv", default=None, help="also write the per-step device-event samples to this CSV file")
    ap.add_argument("--side", default=None,
                    help="comma-separated names of `extra` cases: time only these and print them (one GPU)")
    ap.add_argument("--profile", default=None,
                    choices=["decode", "decode_persistent", "decode_d256", "decode_nz", "config3", "reshape", "reshape_a8", "reshape_d256",
                             "reshape_a8_d256", "lm_decode", "lm_reshape", "scatter", "nz_import"],
                    help="run a small case of one kernel (for ncu), print no bench line")
    args = ap.parse_args()
    if args.profile:
        run_profile_case(args)
    elif args.side:
        import torch
        import ascend_micro_harness_b200 as tq
        torch.cuda.set_device(0)
        print(json.dumps({"side": side_measurements(torch, tq, torch.device("cuda", 0), args)}))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
