#!/usr/bin/env python3
"""Benchmark of the encode path (text -> token ids) on 1..8 B200s of one box.

    python bench.py --gpus N --steps K --warmup W            # this library (libgtok, CUDA)
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU encoder on host cores

A step is one encode of the workload document: the Llama-3-shaped configuration
(seeded synthetic vocabulary of 127,744 merges + 256 special tokens, one ~4.5 MB
document of ~0.9 M tokens; stands in for the real vocabulary and corpus, which are
not available offline).  With N > 1 every rank encodes its own document of that
configuration (weak scaling; documents are independent, the only cross-GPU step
is an all-gather of the per-rank token counts for the global offsets).

`value` is input MB/s (1e6 bytes) with the text already in device memory, timed
with CUDA events around each graph replay on the stream that launches it, L2
flushed between replays; `e2e` is the same through gtok_encode with host buffers
(pinned H2D, replay, D2H inside the timed region).  `decode` (1 GPU) is the way back:
the workload's ids through gtok_x_decode to its bytes.  One JSON line on stdout.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "encode_throughput_1M_token_doc"
UNIT = "MB/s"
WORKLOAD = "config1: Llama-3-shaped BPE (127744 merges, 256 specials), one ~4.5 MB / ~0.9M-token synthetic document"


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w", buffering=1), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def wait_first_sample(self, timeout_s=8.0):
        """nvidia-smi takes a moment to start: block until its first line is there."""
        t0 = time.perf_counter()
        while self.proc and time.perf_counter() - t0 < timeout_s:
            try:
                if os.path.getsize(self.path) > 0:
                    return
            except OSError:
                return
            time.sleep(0.05)

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.remove(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["sm_max_mhz"] = float(max(mx))
        out["reasons"] = sorted(reasons)
        return out


def workload(rank):
    """(tokenizer.json path, document bytes) for this rank."""
    from graphtok_b200 import synth
    path = synth.vocab_path("cfg1")
    vocab, tcfg, seed, nbytes = synth.DOCS[1]
    doc = synth.text(tcfg, seed + 1000 * rank, nbytes)
    return path, doc


def prompt_latency(g, path, want_tokens=131072, reps=40):
    """p50/p90 of gtok_encode (host buffers in and out) on the prefix of the adversarial long-context
    document (configuration 4: base64 blocks, 1-64 KB character repeats, long digit strings, ordinary
    text) that encodes to about 128k tokens."""
    from graphtok_b200 import synth
    _, long_doc = synth.config_doc(4)
    lo, hi = 1 << 16, min(len(long_doc), 4 << 20)
    out = np.empty(hi + 16, dtype=np.uint32)

    def count(nb):
        b = long_doc[:nb]
        return g.lib.gtok_encode(g.handle, b, len(b), out.ctypes.data, out.size)

    while hi - lo > 4096:                      # shortest prefix with at least want_tokens ids
        mid = (lo + hi) // 2
        if count(mid) >= want_tokens:
            hi = mid
        else:
            lo = mid
    prompt = long_doc[:hi]
    n_tok = count(len(prompt))
    ts = []
    for _ in range(reps):
        t = time.perf_counter()
        g.lib.gtok_encode(g.handle, prompt, len(prompt), out.ctypes.data, out.size)
        ts.append(time.perf_counter() - t)
    ts.sort()
    return {"p50_ms": ts[len(ts) // 2] * 1e3, "p90_ms": ts[int(len(ts) * 0.9)] * 1e3, "tokens": int(n_tok), "bytes": len(prompt),
            "what": "gtok_encode with host buffers, prefix of the configuration-4 document (Llama-3-shaped vocabulary)"}


def decode_numbers(g, doc, flush, reps=20):
    """Decoding of the workload's own ids back to its bytes through gtok_x_decode (host buffers):
    CUDA-event time of the decode graph (control-block reset + one kernel) with L2 flushed before
    each call, wall time of the whole call into a pageable and into a page-locked buffer."""
    import ctypes
    import torch
    ids = g.encode(doc)
    out = np.empty(len(doc) + 64, dtype=np.uint8)
    pinned = torch.empty(len(doc) + 64, dtype=torch.uint8).pin_memory().numpy()
    ms = ctypes.c_float(0.0)

    def call(buf):
        t = time.perf_counter()
        n = g.lib.gtok_x_decode(g.handle, ids.ctypes.data, ids.size, buf.ctypes.data, buf.size, None, ctypes.byref(ms))
        return n, (time.perf_counter() - t) * 1e3

    n, _ = call(out)
    if n != len(doc) or out[:n].tobytes() != bytes(doc):
        raise SystemExit("decode(encode(document)) differs from the document")
    graph, wall, wall_pin = [], [], []
    for _ in range(reps):
        flush.zero_()
        torch.cuda.synchronize()
        wall.append(call(out)[1])
        graph.append(ms.value)
        wall_pin.append(call(pinned)[1])
    gm = float(np.median(graph))
    # algorithmic bytes: ids read (4 B each), the bytes written, 8 B of offsets and 16 B of spelling per id
    algo = 4.0 * ids.size + len(doc) + 24.0 * ids.size
    return {"what": "gtok_x_decode of the workload's ids back to its bytes (checked equal)", "ids": int(ids.size), "bytes": len(doc),
            "graph_ms": gm, "ids_per_s": ids.size / (gm * 1e-3), "algorithmic_bytes": algo, "achieved_gbs": algo / (gm * 1e-3) / 1e9,
            "e2e_ms_pageable_output": float(np.median(wall)), "e2e_ms_page_locked_output": float(np.median(wall_pin)), "gpu_launches_per_call": 1}


def small_input_latency(path, doc, reps=60):
    """p50 of gtok_encode (host buffers) on short prefixes of the workload, on a handle created for
    64 KB inputs: what a short prompt costs (launch and phase latency, not bandwidth)."""
    from graphtok_b200 import GTok
    g = GTok(path, max_bytes=64 << 10)
    out = np.empty((64 << 10) + 16, dtype=np.uint32)
    res = {}
    try:
        for nb in (64, 1024, 16384, 65536):
            b = bytes(doc[:nb])
            while b and (b[-1] & 0xC0) == 0x80:       # do not cut a codepoint
                b = b[:-1]
            for _ in range(5):
                g.lib.gtok_encode(g.handle, b, len(b), out.ctypes.data, out.size)
            ts = []
            for _ in range(reps):
                t = time.perf_counter()
                n = g.lib.gtok_encode(g.handle, b, len(b), out.ctypes.data, out.size)
                ts.append(time.perf_counter() - t)
            ts.sort()
            res["%d_bytes" % nb] = {"p50_us": ts[len(ts) // 2] * 1e6, "p90_us": ts[int(len(ts) * 0.9)] * 1e6, "tokens": int(n)}
    finally:
        g.close()
    res["what"] = "gtok_encode with host buffers on prefixes of the workload document, handle created for 64 KB"
    return res


def cpu_encoder(path):
    """The reference's own host encoder when it was built from its sources, else the oracle port."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    if os.path.exists(oracle_lib.REF_SO):
        return oracle_lib.Reference(path), "reference"
    return oracle_lib.Oracle(path), "port"


def time_cpu(enc, doc, budget_s=12.0, max_reps=8):
    """Encodes `doc` repeatedly (at least twice) within the budget: returns (best seconds, runs, tokens)."""
    times, n_tok = [], 0
    t_all = time.perf_counter()
    while len(times) < 2 or (time.perf_counter() - t_all < budget_s and len(times) < max_reps):
        t = time.perf_counter()
        ids = enc.encode_normalized(doc)
        times.append(time.perf_counter() - t)
        n_tok = len(ids)
    return min(times), len(times), n_tok


def run_reference(args, rank, world):
    if rank != 0:
        return
    path, doc = workload(0)
    enc, kind = cpu_encoder(path)
    for _ in range(args.warmup if args.warmup < 2 else 1):
        enc.encode_normalized(doc)
    ts = []
    n_tok = 0
    for _ in range(args.steps):
        t = time.perf_counter()
        n_tok = len(enc.encode_normalized(doc))
        ts.append(time.perf_counter() - t)
    per = float(np.mean(ts))
    val = len(doc) / per / 1e6
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8/u32 integer", "data": "synthetic", "tokens_per_s": n_tok / per,
        "config": {"workload": WORKLOAD, "bytes": len(doc), "tokens": n_tok},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": 1, "kind": kind,
                         "sample": "the whole workload document per step, one host thread (the reference's host encoder is single-threaded per engine)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="gtok", choices=["gtok", "reference"])
    ap.add_argument("--decode-only", action="store_true", help="only the decode figures of the workload (1 GPU; profiling runs of decode_kernel)")
    ap.add_argument("--quick", action="store_true", help="skip the CPU baseline and the prompt-latency section (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "gtok" else args.warmup

    rank = env_int("RANK", 0)
    local_rank = env_int("LOCAL_RANK", 0)
    world = env_int("WORLD_SIZE", 1)

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the encode path has no CPU implementation")
    torch.cuda.set_device(local_rank)
    os.environ["GTOK_DEVICE"] = str(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from graphtok_b200 import GTok
    path, doc = workload(rank)
    g = GTok(path, max_bytes=len(doc) + 4096)
    n_bytes = len(doc)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")   # larger than the 126 MB L2

    if args.decode_only:
        if world > 1:
            raise SystemExit("bench.py --decode-only is a 1-GPU run")
        print(json.dumps({"metric": "decode_of_the_workload_ids", "n_gpus": 1, "decode": decode_numbers(g, doc, flush, reps=max(args.steps, 1))}), flush=True)
        g.close()
        return

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput ------------------------------------
    g.stage(doc)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        flush.zero_()
        torch.cuda.synchronize()
        n_tok, _ = g.replay()
    sampler.wait_first_sample()
    barrier()
    dev_ms = []
    wall0 = time.perf_counter()
    for _ in range(args.steps):
        flush.zero_()
        torch.cuda.synchronize()
        n_tok, ms = g.replay()
        dev_ms.append(ms)
    barrier()
    wall = time.perf_counter() - wall0
    step_ms = float(np.sum(dev_ms)) / args.steps

    # per-kernel times (same kernels launched one by one with events between them)
    prof = []
    for _ in range(max(5, min(args.steps, 20))):
        flush.zero_()
        torch.cuda.synchronize()
        prof.append(g.profile()[1:])
    prof = np.array(prof)
    kern_ms = [float(x) for x in prof[:, :4].mean(axis=0)]     # pretok, words, miss, assemble

    # ---- end to end through the C ABI ------------------------------------
    for _ in range(3):
        ids = g.encode(doc)
    # the caller's output buffer is page-locked (the library then copies the ids straight into it);
    # the same call with an ordinary pageable buffer is timed too and reported beside it
    out_pinned = torch.empty(n_bytes + 16, dtype=torch.int32).pin_memory()
    out = out_pinned.numpy()
    for _ in range(3):
        g.lib.gtok_encode(g.handle, doc, n_bytes, out.ctypes.data, out.size)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        n_e2e = g.lib.gtok_encode(g.handle, doc, n_bytes, out.ctypes.data, out.size)
    barrier()
    e2e_s = (time.perf_counter() - t0) / args.steps
    out_pg = np.empty(n_bytes + 16, dtype=np.uint32)
    for _ in range(3):
        g.lib.gtok_encode(g.handle, doc, n_bytes, out_pg.ctypes.data, out_pg.size)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        g.lib.gtok_encode(g.handle, doc, n_bytes, out_pg.ctypes.data, out_pg.size)
    barrier()
    e2e_pageable_s = (time.perf_counter() - t0) / args.steps
    clocks = sampler.stop()

    # ---- latency of a 128k-token prompt (rank 0 of a 1-GPU run only) -------------
    latency = None
    if world == 1 and not args.quick:
        latency = prompt_latency(g, path)
    decode = decode_numbers(g, doc, flush) if world == 1 and not args.quick else None
    small = small_input_latency(path, doc) if world == 1 and not args.quick else None

    # ---- reduce over ranks ---------------------------------------------------
    stats = torch.tensor([step_ms, e2e_s * 1e3, float(n_bytes), float(n_tok)] + kern_ms, dtype=torch.float64, device="cuda")
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        # the path's one exchange step: per-rank token counts -> global offsets
        counts = [torch.zeros(1, dtype=torch.int64, device="cuda") for _ in range(world)]
        dist.all_gather(counts, torch.tensor([n_tok], dtype=torch.int64, device="cuda"))
        offsets = np.concatenate([[0], np.cumsum([int(c.item()) for c in counts])])
        step_ms, e2e_ms = float(mx[0]), float(mx[1])
        tot_bytes, tot_tok = float(sm[2]), float(sm[3])
        kern_ms = [float(mx[4 + i]) for i in range(4)]
    else:
        e2e_ms = e2e_s * 1e3
        tot_bytes, tot_tok = float(n_bytes), float(n_tok)
        offsets = np.array([0, n_tok])

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        tm, tw, to = g.table_bytes()
        # Algorithmic bytes per launch of each kernel (what it must read and write once):
        #   pretok   : text in, boundary + added-token bits out, class tables
        #   words    : text + bits in, one u32 slot per byte out, whole-word table
        #   miss     : the unknown pre-tokens' bytes in, their ids out, merge table
        #   assemble : one u32 slot per byte in, ids out
        names = ["pretok_kernel", "words_kernel", "miss_kernel", "assemble_kernel"]
        algo_of = {
            "pretok_kernel": n_bytes + 2 * n_bytes / 8.0 + to,
            "words_kernel": n_bytes + 2 * n_bytes / 8.0 + 4.0 * n_bytes + tw,
            "miss_kernel": n_bytes * 0.25 + 4.0 * n_tok * 0.25 + tm,
            "assemble_kernel": 4.0 * n_bytes + 4.0 * n_tok,
        }
        # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures of
        # this workload summarised under profiles/*_kernel_config1.md
        # (the pre-tokenization kernel's figure includes write-back that is not its own, 26.3 MB in this capture:
        # it is the first kernel after the 256 MB L2 flush and the flush's dirty lines leave L2 while it runs)
        traffic_of = {"pretok_kernel": 5.40e6 + 26.26e6, "words_kernel": 12.61e6, "miss_kernel": 13.88e6 + 0.21e6, "assemble_kernel": 18.39e6}
        dom = int(np.argmax(kern_ms))
        algo = algo_of[names[dom]]
        achieved = algo / (kern_ms[dom] * 1e-3) / 1e9
        per_kernel = {k: {"ms": ms, "algorithmic_bytes": algo_of[k], "achieved_gbs": algo_of[k] / (ms * 1e-3) / 1e9,
                          "frac": algo_of[k] / (ms * 1e-3) / 1e9 / peak, "dram_traffic": traffic_of[k]} for k, ms in zip(names, kern_ms)}
        whole = (n_bytes + 4.0 * n_tok + tm + tw + to) / (step_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": tot_bytes / (step_ms * 1e-3) / 1e6, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8/u32 integer", "data": "synthetic",
            "tokens_per_s": tot_tok / (step_ms * 1e-3),
            "config": {"workload": WORKLOAD, "bytes_per_gpu": n_bytes, "tokens_per_gpu": int(n_tok), "l2": "flushed between steps (256 MB write)",
                       "parallelism": "documents sharded across ranks; all_gather of token counts only"},
            "e2e": {"value": tot_bytes / (e2e_ms * 1e-3) / 1e6, "unit": UNIT, "h2d_bytes_per_step": n_bytes + 16, "d2h_bytes_per_step": int(4 * n_tok + 8),
                    "ms_per_step": e2e_ms, "buffers": "input: pageable host bytes; output: page-locked host array",
                    "ms_per_step_pageable_output": e2e_pageable_s * 1e3},
            "gpu_launches": 4 * args.steps * world,
            "kernels_ms": dict(zip(names, kern_ms)),
            "kernels_roofline": per_kernel,
            "roofline": {"bound": "hbm", "kernel": names[dom], "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_kind, "traffic": traffic_of[names[dom]], "algorithmic_bytes": algo,
                         "whole_replay": {"achieved": whole, "frac": whole / peak}},
            "clocks": clocks,
            "latency_128k_prompt": latency,
            "decode": decode,
            "latency_small_inputs": small,
            "wall_s_timed_region": wall,
            "global_token_offsets": [int(x) for x in offsets],
        }
        # CPU baseline on this box's host cores (reported, not a target).
        try:
            if args.quick:
                raise RuntimeError("skipped (--quick)")
            enc, kind = cpu_encoder(path)
            best, runs, cpu_tok = time_cpu(enc, doc)
            line["cpu_baseline"] = {"value": n_bytes / best / 1e6, "unit": UNIT, "cores": 1, "kind": kind,
                                    "sample": "whole workload document, best of %d runs, one host thread" % runs, "tokens_match": bool(cpu_tok == n_tok)}
        except Exception as e:   # the baseline is a report, never a reason to lose the GPU number
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "unavailable", "sample": str(e)[:200]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
