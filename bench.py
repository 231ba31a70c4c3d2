#!/usr/bin/env python3
"""Benchmark of the encode path (text -> token ids) on 1..8 B200s of one box.

    python bench.py --gpus N --steps K --warmup W            # this library (libgtok, CUDA)
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU encoder on host cores

Workload: the Llama-3-shaped configuration (seeded synthetic vocabulary of 127,744 merges + 256
special tokens, one ~4.5 MB document of ~0.9 M tokens; stands in for the real vocabulary and
corpus, which are not available offline).  A step is one encode of that document.  With N > 1 the
SAME document is cut into N parts at positions where a pre-token starts whatever precedes it
(gtok_x_plan_chunks), rank r encodes part r, and the only cross-GPU step is an all-gather of the
per-rank token counts for the global offsets (strong scaling; no data-path collective).  Rank 0
checks the concatenated ids against the reference's CPU encoder before anything is timed.

`value` is input MB/s (1e6 bytes) with the text already in device memory: CUDA events around each
graph replay on the stream that launches it, L2 flushed and left clean between replays (a 256 MB
fill, then a read sweep of a second 256 MB buffer), max over ranks.  `e2e` is the same through
gtok_encode with host buffers (H2D, replay, D2H inside the timed region).  Extra keys give the
other sharded configurations (the 8,192-document batch by documents, the 32 MB adversarial
document by chunks), the 128k-token prompt latency, small-input latency and decoding (1 GPU).
One JSON line on stdout.
"""
import argparse
import ctypes
import json
import os
import re
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
KERNELS = ["pretok_kernel", "words_kernel", "miss_kernel", "assemble_kernel"]


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


def config_dict(n_bytes, n_tok, world):
    """The same keys from both arms, so that the two lines can be matched key by key."""
    return {"workload": WORKLOAD, "bytes": int(n_bytes), "tokens": int(n_tok),
            "l2": "flushed and left clean between steps (256 MB fill, then a 256 MB read sweep)",
            "parallelism": "1 GPU" if world == 1 else "the one document cut into %d pre-token-aligned chunks, one per GPU; all_gather of token counts only" % world}


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
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
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
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def workload():
    """(tokenizer.json path, document bytes): the same on every rank."""
    from graphtok_b200 import synth
    return synth.config_doc(1)


def cpu_encoder(path):
    """The reference's own host encoder when it was built from its sources, else the oracle port."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib
    if os.path.exists(oracle_lib.REF_SO):
        return oracle_lib.Reference(path), "reference"
    return oracle_lib.Oracle(path), "port"


def reference_table_bytes(path):
    """Table bytes one replay reads as the reference lays them out (what the roofline's T_table means):
    merge hash of 2^k >= 2 x merges slots of 16 B (8 B when vocabulary and merges fit 16 bits,
    src/vocab.cc:686-795), for ignore_merges vocabularies its direct table of 2^k >= 2 x vocabulary
    slots of 12 B plus the token bytes (src/vocab.cc:1134-1171), the 17,216-byte class table and the
    1 KiB byte-to-id table."""
    with open(path, encoding="utf-8") as f:
        model = json.load(f)["model"]
    n_merges, n_vocab = len(model["merges"]), len(model["vocab"])
    slots = 16
    while slots < 2 * n_merges:
        slots *= 2
    merge = slots * (8 if (n_merges <= 65535 and n_vocab <= 65535) else 16)
    direct = 0
    if model.get("ignore_merges"):
        dslots = 16
        while dslots < 2 * n_vocab:
            dslots *= 2
        direct = dslots * 12 + sum(len(k) for k in model["vocab"])      # spellings: about a byte per character
    return {"merge": merge, "direct": direct, "class_and_bytes": 17216 + 1024, "total": merge + direct + 17216 + 1024}


def profile_traffic():
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of each kernel from the ncu
    summaries under profiles/, when they were taken from this very source (their `source:` line equals
    the hash of graphtok_b200/csrc); None for a kernel otherwise."""
    from graphtok_b200 import build
    want = build.source_hash()
    out = {}
    for k in KERNELS:
        out[k] = None
        p = os.path.join(ROOT, "profiles", "%s_config1.md" % k)
        try:
            text = open(p).read()
        except OSError:
            continue
        m = re.search(r"^source:\s*([0-9a-f]+)", text, re.M)
        rd = re.search(r"dram__bytes_read\.sum\s*\|?\s*([0-9.eE+]+)\s*(K|M|G)?byte", text)
        wr = re.search(r"dram__bytes_write\.sum\s*\|?\s*([0-9.eE+]+)\s*(K|M|G)?byte", text)
        if not (m and rd and wr) or m.group(1) != want:
            continue
        scale = {None: 1.0, "K": 1e3, "M": 1e6, "G": 1e9}
        out[k] = float(rd.group(1)) * scale[rd.group(2)] + float(wr.group(1)) * scale[wr.group(2)]
    return out


def spread(ms):
    return {"min": float(np.min(ms)), "median": float(np.median(ms)), "max": float(np.max(ms)), "mean": float(np.mean(ms))}


def prompt_latency(g, reps=200, want_tokens=131072):
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
    return {"p50_ms": ts[len(ts) // 2] * 1e3, "p90_ms": ts[int(len(ts) * 0.9)] * 1e3, "calls": reps, "tokens": int(n_tok), "bytes": len(prompt),
            "what": "gtok_encode with host buffers, prefix of the configuration-4 document (Llama-3-shaped vocabulary)"}


def decode_numbers(g, doc, flush, reps=20):
    """Decoding of the workload's own ids back to its bytes through gtok_x_decode (host buffers):
    CUDA-event time of the decode graph with L2 flushed before each call, wall time of the whole call
    into a pageable and into a page-locked buffer."""
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
        flush()
        wall.append(call(out)[1])
        graph.append(ms.value)
        wall_pin.append(call(pinned)[1])
    gm = float(np.median(graph))
    # algorithmic bytes: ids read (4 B each), the bytes written, 8 B of offsets and 16 B of spelling per id
    algo = 4.0 * ids.size + len(doc) + 24.0 * ids.size
    return {"what": "gtok_x_decode of the workload's ids back to its bytes (checked equal)", "ids": int(ids.size), "bytes": len(doc),
            "graph_ms": gm, "ids_per_s": ids.size / (gm * 1e-3), "algorithmic_bytes": algo, "achieved_gbs": algo / (gm * 1e-3) / 1e9,
            "e2e_ms_pageable_output": float(np.median(wall)), "e2e_ms_page_locked_output": float(np.median(wall_pin)), "gpu_launches_per_call": 1}


def small_input_latency(path, doc, enc, reps=60):
    """p50 of gtok_encode (host buffers) on short prefixes of the workload, on a handle created for 64 KB
    inputs and on one created for 8 MiB (what a serving process keeps), beside the reference's CPU
    encoder on the same prefixes: what a short prompt costs, and where the two cross."""
    from graphtok_b200 import GTok
    res = {"what": "gtok_encode with host buffers on prefixes of the workload document; cpu = the reference's host encoder on this box, one thread"}
    prefixes = {}
    for nb in (64, 1024, 4096, 16384, 65536):
        b = bytes(doc[:nb])
        while b and (b[-1] & 0xC0) == 0x80:       # do not cut a codepoint
            b = b[:-1]
        prefixes[nb] = b
    for label, cap in (("handle_64KB", 64 << 10), ("handle_8MiB", 8 << 20)):
        g = GTok(path, max_bytes=cap)
        out = np.empty((64 << 10) + 16, dtype=np.uint32)
        rows = {}
        try:
            for nb, b in prefixes.items():
                for _ in range(5):
                    g.lib.gtok_encode(g.handle, b, len(b), out.ctypes.data, out.size)
                ts = []
                for _ in range(reps):
                    t = time.perf_counter()
                    n = g.lib.gtok_encode(g.handle, b, len(b), out.ctypes.data, out.size)
                    ts.append(time.perf_counter() - t)
                ts.sort()
                rows["%d_bytes" % nb] = {"p50_us": ts[len(ts) // 2] * 1e6, "p90_us": ts[int(len(ts) * 0.9)] * 1e6, "tokens": int(n)}
        finally:
            g.close()
        res[label] = rows
    cpu = {}
    for nb, b in prefixes.items():
        ts = []
        for _ in range(20):
            t = time.perf_counter()
            enc.encode_normalized(b)
            ts.append(time.perf_counter() - t)
        ts.sort()
        cpu["%d_bytes" % nb] = {"p50_us": ts[len(ts) // 2] * 1e6}
    res["cpu"] = cpu
    cross = None
    for nb in sorted(prefixes):
        if res["handle_8MiB"]["%d_bytes" % nb]["p50_us"] <= cpu["%d_bytes" % nb]["p50_us"]:
            cross = nb
            break
    res["gpu_not_slower_from_bytes"] = cross
    return res


def time_cpu(enc, doc, budget_s=12.0, max_reps=8):
    """Encodes `doc` repeatedly (at least twice) within the budget: returns (best seconds, runs, ids)."""
    times, ids = [], None
    t_all = time.perf_counter()
    while len(times) < 2 or (time.perf_counter() - t_all < budget_s and len(times) < max_reps):
        t = time.perf_counter()
        ids = enc.encode_normalized(doc)
        times.append(time.perf_counter() - t)
    return min(times), len(times), ids


def run_reference(args, rank, world):
    if rank != 0:
        return
    path, doc = workload()
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
        "warmup": args.warmup, "ms_per_step": per * 1e3, "ms_per_step_spread": spread(np.array(ts) * 1e3), "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "u8/u32 integer", "data": "synthetic", "tokens_per_s": n_tok / per,
        "config": config_dict(len(doc), n_tok, args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": 1, "kind": kind,
                         "sample": "the whole workload document per step, one host thread (the reference's host encoder is single-threaded per engine)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="gtok", choices=["gtok", "reference"])
    ap.add_argument("--decode-only", action="store_true", help="only the decode figures of the workload (1 GPU; profiling runs of decode_kernel)")
    ap.add_argument("--quick", action="store_true", help="skip the CPU baseline, the latency sections and the other configurations (profiling runs)")
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

    from graphtok_b200 import GTok, plan_documents, synth
    path, doc = workload()
    fill = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")    # larger than the 126 MB L2
    sweep = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")    # a second 256 MB, only ever read

    def flush():
        """L2 holds none of the workload afterwards and no dirty lines: the fill evicts, the read sweep
        pushes the fill's dirty lines out, so that the first timed kernel does not pay their write-back."""
        fill.zero_()
        sweep.sum()
        torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def all_max(x):
        t = torch.tensor(x, dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def gather_counts(n):
        """The path's one exchange step: per-rank token counts -> int64 global offsets."""
        if world == 1:
            return np.array([0, n], dtype=np.int64)
        counts = [torch.zeros(1, dtype=torch.int64, device="cuda") for _ in range(world)]
        dist.all_gather(counts, torch.tensor([n], dtype=torch.int64, device="cuda"))
        return np.concatenate([[0], np.cumsum([int(c.item()) for c in counts])]).astype(np.int64)

    def gather_ids(ids, offsets):
        """Every rank's ids on rank 0 (outside any timed region)."""
        if world == 1:
            return ids
        width = int(np.max(np.diff(offsets)))
        mine = torch.zeros(width, dtype=torch.int32, device="cuda")
        mine[:ids.size] = torch.from_numpy(ids.astype(np.int32)).cuda()
        parts = [torch.zeros(width, dtype=torch.int32, device="cuda") for _ in range(world)]
        dist.all_gather(parts, mine)
        if rank != 0:
            return None
        return np.concatenate([p.cpu().numpy()[:int(offsets[r + 1] - offsets[r])].astype(np.uint32) for r, p in enumerate(parts)])

    if args.decode_only:
        if world > 1:
            raise SystemExit("bench.py --decode-only is a 1-GPU run")
        g = GTok(path, max_bytes=len(doc) + 4096)
        print(json.dumps({"metric": "decode_of_the_workload_ids", "n_gpus": 1, "decode": decode_numbers(g, doc, flush, reps=max(args.steps, 1))}), flush=True)
        g.close()
        return

    # ---- this rank's part of the one document --------------------------------------
    planner = GTok(path, max_bytes=4096)                 # the planner only reads the vocabulary's family
    cuts = planner.plan_chunks(doc, world) if world > 1 else np.array([0, len(doc)], dtype=np.uint64)
    planner.close()
    part = doc[int(cuts[rank]):int(cuts[rank + 1])]
    shard_bytes = np.diff(cuts.astype(np.int64))
    g = GTok(path, max_bytes=len(part) + 4096)
    n_bytes = len(doc)

    # ---- parity gate: ids, not counts, against the reference's CPU encoder, before any timing ----
    ids_part = g.encode(part)
    offsets = gather_counts(ids_part.size)
    ids_all = gather_ids(ids_part, offsets)
    enc = kind = cpu_ids = None
    if rank == 0:
        enc, kind = cpu_encoder(path)
        cpu_ids = enc.encode_normalized(doc)
        if not np.array_equal(ids_all, cpu_ids):
            raise SystemExit("bench.py: ids differ from the %s CPU encoder (%d vs %d ids): nothing timed" % (kind, ids_all.size, cpu_ids.size))
    n_tok_total = int(offsets[-1])

    # ---- device-resident throughput ------------------------------------
    g.stage(part)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        flush()
        g.replay()
    sampler.wait_first_sample()
    barrier()
    dev_ms = []
    wall0 = time.perf_counter()
    for _ in range(args.steps):
        flush()
        n_tok, ms = g.replay()
        dev_ms.append(ms)
    barrier()
    wall = time.perf_counter() - wall0
    stats = g.work_stats()

    # per-kernel times (same kernels launched one by one with events between them)
    prof = []
    for _ in range(max(5, min(args.steps, 20))):
        flush()
        prof.append(g.profile()[1:])
    prof = np.array(prof)
    kern_ms = [float(x) for x in prof[:, :4].mean(axis=0)]     # pretok, words, miss, assemble

    # ---- end to end through the C ABI ------------------------------------
    # host buffers in three combinations: text and ids both in page-locked memory (what a serving
    # process that owns its buffers gives the library: the device reads and writes them directly), ordinary
    # pageable text into page-locked ids, and both pageable (staged through the handle's pinned buffers)
    out_pinned = torch.empty(len(part) + 16, dtype=torch.int32).pin_memory()
    out = out_pinned.numpy()
    out_pg = np.empty(len(part) + 16, dtype=np.uint32)
    in_pinned = torch.frombuffer(bytearray(part), dtype=torch.uint8).pin_memory()
    in_pin_ptr = ctypes.c_void_p(in_pinned.data_ptr())
    variants = (("pinned", in_pin_ptr, out), ("pageable_in", part, out), ("pageable", part, out_pg))
    e2e = {label: [] for label, _, _ in variants}
    for label, src, buf in variants:
        for _ in range(max(3, args.warmup)):
            g.lib.gtok_encode(g.handle, src, len(part), buf.ctypes.data, buf.size)
    barrier()
    # the three variants take turns inside every step, so that whatever else the host is doing at the
    # moment (other tenants, clock sampling) falls on all of them alike
    for _ in range(args.steps):
        for label, src, buf in variants:
            t = time.perf_counter()
            n_e2e = g.lib.gtok_encode(g.handle, src, len(part), buf.ctypes.data, buf.size)
            e2e[label].append((time.perf_counter() - t) * 1e3)
            if n_e2e != ids_part.size:
                raise SystemExit("bench.py: the end-to-end call returned %d ids, expected %d" % (n_e2e, ids_part.size))
    barrier()
    for label, src, buf in variants:
        g.lib.gtok_encode(g.handle, src, len(part), buf.ctypes.data, buf.size)
        if not np.array_equal(buf[:ids_part.size].view(np.uint32), ids_part):
            raise SystemExit("bench.py: the end-to-end call returned other ids than the checked ones")
    clocks = sampler.stop()

    # ---- the other sharded configurations (every N), latency and decoding (1 GPU) ----------
    others = None
    if not args.quick:
        others = {}
        # configuration 2: 8,192 documents sharded by documents
        bpath, blob, boffs = synth.config_batch()
        dcut = plan_documents(boffs, world)
        lo_d, hi_d = int(dcut[rank]), int(dcut[rank + 1])
        sub = boffs[lo_d:hi_d + 1].astype(np.int64)
        sub_blob = blob[int(sub[0]):int(sub[-1])]
        sub_offs = (sub - sub[0]).astype(np.uint32)
        gb = GTok(bpath, max_bytes=len(sub_blob) + 4096)
        ids_b, doc_b = gb.encode_batch(sub_blob, sub_offs)
        goffs = gather_counts(ids_b.size)                      # int64 global token offsets of the ranks' ranges
        ids_b_all = gather_ids(ids_b, goffs)
        gb.stage(sub_blob, sub_offs)
        for _ in range(3):
            flush()
            gb.replay()
        barrier()
        bms = []
        for _ in range(max(5, args.steps // 5)):
            flush()
            bms.append(gb.replay()[1])
        barrier()
        # end to end through gtok_encode_batch with host buffers (ids into a page-locked array)
        b_out = torch.empty(len(sub_blob) + 16, dtype=torch.int32).pin_memory().numpy()
        b_doc = np.empty(sub_offs.size, dtype=np.uint32)
        reps_b = max(5, args.steps // 5)
        for _ in range(2):
            gb.lib.gtok_encode_batch(gb.handle, sub_blob, sub_offs.ctypes.data, sub_offs.size - 1, b_out.ctypes.data, b_out.size, b_doc.ctypes.data)
        barrier()
        tb = []
        for _ in range(reps_b):
            t0 = time.perf_counter()
            gb.lib.gtok_encode_batch(gb.handle, sub_blob, sub_offs.ctypes.data, sub_offs.size - 1, b_out.ctypes.data, b_out.size, b_doc.ctypes.data)
            tb.append(time.perf_counter() - t0)
        barrier()
        b_e2e = float(np.mean(tb)) * 1e3
        gb.close()
        b_dev, b_e2e = all_max([float(np.mean(bms)), b_e2e])
        ok_b = None
        if rank == 0:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import oracle_lib
            want_b, _ = oracle_lib.Oracle(bpath).encode_batch(blob, boffs)
            ok_b = bool(np.array_equal(ids_b_all, want_b))
        others["config2_batch_8192_docs"] = {
            "bytes": len(blob), "documents": int(boffs.size - 1), "tokens": int(goffs[-1]), "sharding": "contiguous document ranges of about equal bytes (gtok_x_plan_documents)",
            "device_ms": b_dev, "device_MBps": len(blob) / (b_dev * 1e-3) / 1e6, "e2e_ms": b_e2e, "e2e_MBps": len(blob) / (b_e2e * 1e-3) / 1e6,
            "global_token_offsets_int64": [int(x) for x in goffs], "ids_match_cpu_oracle": ok_b}
        # configuration 4: the 32 MB adversarial document cut into chunks
        _, doc4 = synth.config_doc(4)
        pl = GTok(path, max_bytes=4096)
        cuts4 = pl.plan_chunks(doc4, world) if world > 1 else np.array([0, len(doc4)], dtype=np.uint64)
        pl.close()
        part4 = doc4[int(cuts4[rank]):int(cuts4[rank + 1])]
        g4 = GTok(path, max_bytes=len(part4) + 4096)
        g4.stage(part4)
        for _ in range(3):
            flush()
            n4, _ = g4.replay()
        barrier()
        ms4 = []
        for _ in range(max(5, args.steps // 5)):
            flush()
            ms4.append(g4.replay()[1])
        barrier()
        g4.close()
        off4 = gather_counts(n4)
        d4 = all_max([float(np.mean(ms4))])[0]
        sb4 = np.diff(cuts4.astype(np.int64))
        others["config4_adversarial_32MB"] = {
            "bytes": len(doc4), "tokens": int(off4[-1]), "device_ms": d4, "device_MBps": len(doc4) / (d4 * 1e-3) / 1e6,
            "shard_bytes": [int(x) for x in sb4], "shard_imbalance": float(sb4.max() / sb4.mean()),
            "verified": "token total only (ids at this size are compared with the oracle in tests/test_gpu_parity.py)", "tokens_expected": 14358917}
        # beyond the five configurations: a DeepSeek-V3-shaped vocabulary (three Split patterns, 100,000 merges) on a
        # 4 MiB multilingual document, cut into chunks like configuration 1; ids against the CPU oracle
        path5, doc5 = synth.config_doc(5)
        pl = GTok(path5, max_bytes=4096)
        cuts5 = pl.plan_chunks(doc5, world) if world > 1 else np.array([0, len(doc5)], dtype=np.uint64)
        pl.close()
        part5 = doc5[int(cuts5[rank]):int(cuts5[rank + 1])]
        g5 = GTok(path5, max_bytes=len(part5) + 4096)
        ids5 = g5.encode(part5)
        off5 = gather_counts(ids5.size)
        ids5_all = gather_ids(ids5, off5)
        g5.stage(part5)
        for _ in range(3):
            flush()
            g5.replay()
        barrier()
        ms5 = []
        for _ in range(max(5, args.steps // 5)):
            flush()
            ms5.append(g5.replay()[1])
        barrier()
        g5.close()
        d5 = all_max([float(np.mean(ms5))])[0]
        ok5 = None
        if rank == 0:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import oracle_lib
            ok5 = bool(np.array_equal(ids5_all, oracle_lib.Oracle(path5).encode(doc5)))
        others["deepseek_v3_shaped_4MiB"] = {
            "bytes": len(doc5), "tokens": int(off5[-1]), "device_ms": d5, "device_MBps": len(doc5) / (d5 * 1e-3) / 1e6,
            "ids_match_cpu_oracle": ok5}

    latency = decode = small = None
    if world == 1 and not args.quick:
        latency = prompt_latency(g)
        decode = decode_numbers(g, doc, flush)
        small = small_input_latency(path, doc, enc)

    # ---- reduce over ranks ---------------------------------------------------
    red = all_max([float(np.mean(dev_ms)), float(np.mean(e2e["pinned"])), float(np.mean(e2e["pageable"])), float(np.mean(e2e["pageable_in"]))] + kern_ms)
    step_ms, e2e_ms, e2e_pg_ms, e2e_pgin_ms = red[0], red[1], red[2], red[3]
    kern_max = red[4:8]

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        tm, tw, to = g.table_bytes()
        ref_tab = reference_table_bytes(path)
        n_part = len(part)
        # Algorithmic bytes per launch of each kernel on this rank's part (what it must read and write once;
        # tables at the sizes the reference defines for them, this build's own larger tables beside):
        #   pretok   : text in, boundary + added-token bits out (2 bits per byte), class tables
        #   words    : text + bits in, one u32 slot per byte out, the direct-token table
        #   miss     : the unknown pre-tokens' bytes in (counted from the kernel's own lists), their ids out, merge table
        #   assemble : one u32 slot per byte in, ids out
        miss_bytes = stats["unknown_bytes"] + stats["long_bytes"]
        algo_of = {
            "pretok_kernel": n_part + 2 * n_part / 8.0 + ref_tab["class_and_bytes"],
            "words_kernel": n_part + 2 * n_part / 8.0 + 4.0 * n_part + ref_tab["direct"],
            "miss_kernel": miss_bytes + 4.0 * stats["ids_from_miss_kernel"] + ref_tab["merge"],
            "assemble_kernel": 4.0 * n_part + 4.0 * ids_part.size,
        }
        own_tables_of = {"pretok_kernel": to, "words_kernel": tw, "miss_kernel": tm, "assemble_kernel": 0}
        traffic_of = profile_traffic() if world == 1 else {k: None for k in KERNELS}
        dom = int(np.argmax(kern_ms))
        per_kernel = {}
        for k, ms in zip(KERNELS, kern_ms):
            per_kernel[k] = {"ms": ms, "algorithmic_bytes": algo_of[k], "achieved_gbs": algo_of[k] / (ms * 1e-3) / 1e9,
                             "frac": algo_of[k] / (ms * 1e-3) / 1e9 / peak, "own_table_bytes": own_tables_of[k], "dram_traffic": traffic_of[k]}
        dk = KERNELS[dom]
        whole_algo = n_bytes + 4.0 * n_tok_total + ref_tab["total"]
        whole = whole_algo / (step_ms * 1e-3) / 1e9
        whole_own = (n_bytes + 4.0 * n_tok_total + tm + tw + to) / (step_ms * 1e-3) / 1e9
        whole_notab = (n_bytes + 4.0 * n_tok_total) / (step_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": n_bytes / (step_ms * 1e-3) / 1e6, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_ms, "ms_per_step_spread_rank0": spread(dev_ms), "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "u8/u32 integer", "data": "synthetic",
            "tokens_per_s": n_tok_total / (step_ms * 1e-3),
            "config": config_dict(n_bytes, n_tok_total, world),
            "shard_bytes": [int(x) for x in shard_bytes], "shard_imbalance": float(shard_bytes.max() / shard_bytes.mean()),
            "parity": {"checked": "ids of the timed workload (all ranks' parts concatenated) against the CPU encoder, before timing", "against": kind, "ids_match": True},
            "e2e": {"value": n_bytes / (e2e_ms * 1e-3) / 1e6, "unit": UNIT, "h2d_bytes_per_step": n_bytes + 16 * world, "d2h_bytes_per_step": int(4 * n_tok_total + 8 * world),
                    "ms_per_step": e2e_ms, "ms_per_step_spread_rank0": spread(e2e["pinned"]), "buffers": "text and ids both in page-locked host memory",
                    "ms_per_step_pageable_input": e2e_pgin_ms, "ms_per_step_pageable_input_and_output": e2e_pg_ms},
            "gpu_launches": 4 * args.steps * world,
            "kernels_ms": dict(zip(KERNELS, kern_ms)), "kernels_ms_max_over_ranks": dict(zip(KERNELS, kern_max)),
            "kernels_roofline": per_kernel,
            "work": stats,
            "roofline": {"bound": "hbm", "kernel": dk, "achieved": per_kernel[dk]["achieved_gbs"], "peak": peak, "unit": "GB/s", "frac": per_kernel[dk]["frac"],
                         "peak_source": peak_kind, "traffic": traffic_of[dk], "algorithmic_bytes": algo_of[dk],
                         "whole_replay": {"algorithmic_bytes": whole_algo, "achieved": whole, "frac": whole / peak,
                                          "what": "text + 4 B per id + tables at the reference's sizes (merge hash, direct table and spellings, class table), over the replay time"},
                         "whole_replay_own_tables": {"achieved": whole_own, "frac": whole_own / peak, "table_bytes": tm + tw + to},
                         "whole_replay_without_tables": {"achieved": whole_notab, "frac": whole_notab / peak},
                         "reference_table_bytes": ref_tab},
            "clocks": clocks,
            "other_configurations": others,
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
            best, runs, ids_cpu = time_cpu(enc, doc)
            line["cpu_baseline"] = {"value": n_bytes / best / 1e6, "unit": UNIT, "cores": 1, "kind": kind,
                                    "sample": "whole workload document, best of %d runs, one host thread" % runs, "ids_match": bool(np.array_equal(ids_cpu, ids_all))}
        except Exception as e:   # the baseline is a report, never a reason to lose the GPU number
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "unavailable", "sample": str(e)[:200]}
        print(json.dumps(line), flush=True)
    g.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
