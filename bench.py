#!/usr/bin/env python
"""Decode-attention benchmark of the PQ-HSA per-step operator on B200.

One "step" = one layer-step of the hot path over one batch: append one K/V row
per stream, encode the key that leaves the local window into the index, and run
the hybrid decode attention (tables, code scan, exact top-k, exact attention over
sink / local / selected rows read in place from the KV cache, per-list background,
one softmax).  KV heads are sharded across the ranks (vLLM tensor-parallel
layout); the only collective is the all-gather of the output slices.

  python bench.py --gpus 1 --steps 300 --warmup 20            # this library
  python bench.py --impl reference --steps 3 --warmup 1       # CPU port of the reference path

Prints ONE JSON line (rank 0).  Timing: CUDA events on the launching stream around
every step, the L2 is flushed (256 MiB written, then 256 MiB read) between timed steps,
queries rotate.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from pqhsa_release_b200 import workloads  # noqa: E402

METRIC = "decode_attention_keys_scanned_per_s"
UNIT = "keys/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(workloads.WORKLOADS) + ["encode_bulk"])
    ap.add_argument("--context", type=int, default=None, help="override the context length (debugging)")
    ap.add_argument("--batch", type=int, default=None, help="override the batch size (debugging)")
    ap.add_argument("--layers", type=int, default=None, help="layers of workload c4 (default 80)")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--flush", default="write+read", choices=["write+read", "write", "read", "none"],
                    help="how the L2 is flushed between timed steps")
    ap.add_argument("--stages", action="store_true", help="also print the per-stage timing table to stderr")
    ap.add_argument("--no-sidecar", action="store_true", help="skip the second end-to-end figure (through GQASidecar)")
    return ap.parse_args()


def profiled_traffic(kernel: str):
    """DRAM bytes (read + written) of one launch of ``kernel`` on workload c2, from the line
    ``dram bytes per launch: <kernel> <bytes>`` of the committed ncu summary; None if the file or the line is missing."""
    import re

    try:
        text = (ROOT / "profiles" / "decode_step_c2_ncu_full.md").read_text()
    except OSError:
        return None
    m = re.search(rf"^dram bytes per launch: {re.escape(kernel)} (\d+)\s*$", text, re.M)
    return int(m.group(1)) if m else None


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# --------------------------------------------------------------------------
# clocks during the timed region (NVML, read-only)
# --------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for b, name in self.REASONS.items():
                    if bits & b:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()
        med = sorted(self.samples)[len(self.samples) // 2] if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# --------------------------------------------------------------------------
# set-up of this library's arm
# --------------------------------------------------------------------------
def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def build_b200(wl, rank, world, device, total_steps, nq=8):
    from pqhsa_release_b200.config import paper_index_config
    from pqhsa_release_b200.device_index import DeviceIndexPool
    from pqhsa_release_b200.index_build import build_index_batch

    hl = wl.kv_heads // world
    heads = range(rank * hl, (rank + 1) * hl)
    S, G, D = wl.batch * hl, wl.group, wl.head_dim
    ctx = wl.context
    sink_end = min(wl.sink_tokens, ctx)
    n0 = wl.retrieval_len()
    margin = total_steps + 64
    pool = DeviceIndexPool(
        num_streams=S, group=G, dtype=wl.dtype, device=device, slot_capacity=n0 + margin,
        num_lists=wl.num_lists, sink_tokens=wl.sink_tokens, local_window=wl.local_window,
        scale=1.0 / math.sqrt(D), top_fraction=wl.top_fraction, tail_capacity=margin,
        max_full=wl.sink_tokens + wl.local_window + 64,
    )
    kc = torch.zeros(wl.batch, hl, ctx + margin, D, dtype=wl.dtype, device=device)
    vc = torch.zeros_like(kc)
    icfg = paper_index_config(num_lists=wl.num_lists)
    for b in range(wl.batch):
        for j, h in enumerate(heads):
            k, v = workloads.mixture_kv(100_000 * b + h, 1, ctx, dtype=wl.dtype, device=device)
            kc[b, j, :ctx], vc[b, j, :ctx] = k[0], v[0]
        idx = build_index_batch(kc[b, :, sink_end : sink_end + n0], vc[b, :, sink_end : sink_end + n0], icfg)
        for j, h in enumerate(heads):
            pool.load_stream(b * hl + j, idx[j], seq_len=ctx, req=b, kv_head=j)
        del idx
    pool.bind_kv_contiguous(kc, vc)
    # rotating inputs: nq query batches planted near random keys, nq new K/V rows
    qs, nks, nvs = [], [], []
    for i in range(nq):
        qb = torch.empty(wl.batch, hl * G, D, dtype=wl.dtype, device=device)
        for b in range(wl.batch):
            qb[b] = workloads.planted_queries(7_000 + 100 * i + b + 31 * rank, kc[b, :, :ctx], G)
        qs.append(qb.reshape(S, G, D).contiguous())
        g = torch.Generator(device=device).manual_seed(9_000 + i + 77 * rank)
        nks.append(torch.randn(S, D, generator=g, device=device).to(wl.dtype))
        nvs.append(torch.randn(S, D, generator=g, device=device).to(wl.dtype))
    return pool, (kc, vc), qs, nks, nvs


class StepRunner:
    """The step as a user issues it: static input buffers, one CUDA graph replay."""

    def __init__(self, pool, wl, world, use_graph, headroom):
        self.pool, self.world = pool, world
        S, G, D = pool.S, pool.G, wl.head_dim
        dev = pool.device
        # the step's inputs sit in one buffer (query rows, new K rows, new V rows): one host-to-device copy per step
        self.inbuf = torch.zeros(S * G * D + 2 * S * D, dtype=wl.dtype, device=dev)
        self.q = self.inbuf[: S * G * D].view(S, G, D)
        self.nk = self.inbuf[S * G * D : S * G * D + S * D].view(S, D)
        self.nv = self.inbuf[S * G * D + S * D :].view(S, D)
        self.out = torch.zeros(S, G, D, dtype=wl.dtype, device=dev)
        self.gathered = torch.zeros(world, S, G, D, dtype=wl.dtype, device=dev) if world > 1 else None
        self.exchange, self.steps_done = None, 0
        if world > 1 and os.environ.get("PQHSA_EXCHANGE", "peer") == "peer":
            # rows stored straight into every rank's buffer by the combine kernel; NCCL otherwise.  The ranks
            # agree on the outcome: one rank without symmetric memory sends all of them to the NCCL form.
            why = ""
            try:
                from pqhsa_release_b200.parallel import PeerExchange

                self.exchange = PeerExchange(pool)
            except Exception as e:  # noqa: BLE001
                why = f"{type(e).__name__}: {e}"
                self.exchange = None
            ok = torch.tensor([1 if self.exchange is not None else 0], dtype=torch.int32, device=dev)
            torch.distributed.all_reduce(ok, op=torch.distributed.ReduceOp.MIN)
            if int(ok.item()) == 0:
                if self.exchange is not None or why:
                    print(f"[bench] peer exchange unavailable on some rank ({why or 'elsewhere'}); using the NCCL all-gather",
                          file=sys.stderr)
                self.exchange = None
                pool.p.peer_world = 0
        self.graph = None
        # tables + thresholds + append + encode, scan, selection (two launches when a row's selection is shared by
        # several CTAs), attend + background, combine (+ the receiving kernel when sharded)
        self.launches_per_step = 5 + (1 if pool.layout.parts > 1 else 0)
        pool.graph_headroom = headroom
        if use_graph:
            self._body()  # warm the lazy set-up (shared-memory opt-in, NCCL) outside the capture
            self.steps_done += 1
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._body()
            pool.note_replayed(appends=-1, encodes=-1)  # the capture pass ran no kernels

    def _body(self):
        p = self.pool
        p.decode_step_append(self.q, self.nk, self.nv, encode=1, out=self.out)
        if self.exchange is not None:
            self.exchange.wait()
        elif self.gathered is not None:
            torch.distributed.all_gather_into_tensor(self.gathered, self.out)

    def step(self):
        if self.graph is None:
            self._body()
        else:
            self.graph.replay()
            self.pool.note_replayed(appends=1, encodes=1)
        self.steps_done += 1

    def result(self):
        """The step's output on this rank: all ranks' rows when sharded."""
        if self.exchange is not None:
            return self.exchange.result(self.steps_done)
        return self.gathered if self.gathered is not None else self.out


def sidecar_e2e(wl, kv, qs, nks, nvs, n_ctx, steps, flush_l2, device):
    """The same step through ``GQASidecar`` as the reference's decode runtime drives it (one sidecar for the
    layer's requests): per step the host copies the queries and the new K/V rows from pinned memory, calls
    ``lean_append`` and ``forward`` (one fused library call, replayed as a self-validated CUDA graph) and reads
    the context back into pinned memory."""
    from pqhsa_release_b200.config import paper_attention_config, paper_index_config
    from pqhsa_release_b200.gqa_sidecar import GQASidecar

    kc, vc = kv
    B, H, G, D = wl.batch, kc.shape[1], wl.group, wl.head_dim
    side = GQASidecar(
        paper_index_config(num_lists=wl.num_lists),
        paper_attention_config(scale=1.0 / math.sqrt(D), sink_tokens=wl.sink_tokens, local_window=wl.local_window,
                               retrieval_top_fraction=wl.top_fraction, index_update_interval=1,
                               index_update_strategy="incremental"),
        num_query_heads=H * G, num_kv_heads=H)
    side.build_cache(kc[:, :, : wl.context], vc[:, :, : wl.context])
    nq = len(qs)
    # the step's inputs go with ONE copy from pinned memory into the sidecar's static input buffer (queries, keys, values)
    dq, dk, dv, flat = side.static_inputs()
    hin = [torch.cat([q.reshape(-1), k.reshape(-1), v.reshape(-1)]).cpu().pin_memory() for q, k, v in zip(qs, nks, nvs)]
    hout = torch.empty(B, H * G, D, dtype=wl.dtype).pin_memory()

    def step(i, ev=None):
        flush_l2()
        if ev is not None:
            ev[0].record()
        flat.copy_(hin[i % nq], non_blocking=True)
        if not side.lean_append(dk, dv, dq):
            raise SystemExit("GQASidecar.lean_append refused one token per request")
        hout.copy_(side.forward(dq), non_blocking=True)
        if ev is not None:
            ev[1].record()

    for i in range(4):
        step(i)
    torch.cuda.synchronize()
    if not bool(torch.isfinite(hout.float()).all()):
        raise SystemExit("sidecar end-to-end check failed: non-finite context")
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for i in range(steps):
        step(4 + i, evs[i])
    torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in evs) / steps
    keys = wl.batch * wl.kv_heads * n_ctx
    out = {"value": keys / (ms / 1e3), "unit": UNIT, "us_per_layer_step": 1e3 * ms, "steps": steps,
           "cuda_graph_active": bool(side.cuda_graph_active),
           "h2d_bytes_per_step": hin[0].numel() * hin[0].element_size(),
           "d2h_bytes_per_step": hout.numel() * hout.element_size(),
           "entry": "GQASidecar.static_inputs + lean_append + forward: one pinned-memory copy in, graph replay, one copy out"}
    del side
    torch.cuda.empty_cache()
    return out


def run_b200(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU port)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    wl = workloads.WORKLOADS[args.workload]
    if args.context or args.batch:
        from dataclasses import replace

        wl = replace(wl, context=args.context or wl.context, batch=args.batch or wl.batch,
                     name=wl.name + " (overridden)")
    if wl.kv_heads % world:
        raise SystemExit(f"{wl.kv_heads} KV heads do not shard over {world} ranks")
    K, W = args.steps, max(args.warmup, 3)
    total_steps = 2 * (K + W) + 16
    t0 = time.time()
    pool, kv, qs, nks, nvs = build_b200(wl, rank, world, device, total_steps)
    runner = StepRunner(pool, wl, world, not args.no_graph, headroom=total_steps + 64)
    setup_s = time.time() - t0
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    flush_rd = torch.zeros(64 << 20, dtype=torch.int32, device=device)

    align_t = torch.zeros(1, dtype=torch.int32, device=device)

    def flush_l2():
        # evict everything: write 256 MiB, then read another 256 MiB so that the L2 is left
        # holding clean lines (a cold cache without a write-back storm under the next kernel)
        if args.flush in ("write", "write+read"):
            flush.zero_()
        if args.flush in ("read", "write+read"):
            flush_rd.sum()
        if world > 1:
            # The flush is part of the measurement, not of the workload: line the ranks up again behind it
            # (a 4-byte all-reduce on the same stream, outside the timed region), so that a step's time does
            # not include waiting for a rank whose flush ran a little longer.
            torch.distributed.all_reduce(align_t)
    nq = len(qs)

    def load_inputs(i):
        runner.q.copy_(qs[i % nq]); runner.nk.copy_(nks[i % nq]); runner.nv.copy_(nvs[i % nq])

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------
    for i in range(W):
        load_inputs(i); flush_l2(); runner.step()
    barrier()
    if runner.exchange is not None:
        # once, outside the timed region: what arrived through the peer stores equals an NCCL all-gather
        check = torch.empty(world, *runner.out.shape, dtype=runner.out.dtype, device=device)
        torch.distributed.all_gather_into_tensor(check.view(world * runner.out.shape[0], *runner.out.shape[1:]), runner.out)
        torch.cuda.synchronize()
        if runner.exchange.timed_out() or not torch.equal(check.view(world, -1, wl.head_dim), runner.result()):
            raise SystemExit("peer exchange check failed: rows differ from the NCCL all-gather (or the flag wait ran out)")
    n_start = int(pool.h_sorted[0] + pool.h_tail[0])
    sampler = ClockSampler(physical_gpu_index(local_rank))
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    sampler.start()
    wall0 = time.perf_counter()
    for i in range(K):
        load_inputs(i); flush_l2()
        ev[i][0].record(); runner.step(); ev[i][1].record()
    barrier()
    wall = time.perf_counter() - wall0
    clocks = sampler.stop()
    total_ms = sum(a.elapsed_time(b) for a, b in ev)

    # ---- end to end through the public call with host buffers --------------
    hin = [torch.cat([qs[i].reshape(-1), nks[i].reshape(-1), nvs[i].reshape(-1)]).cpu().pin_memory() for i in range(nq)]
    res_t = runner.result()
    hout = torch.empty(res_t.shape, dtype=res_t.dtype).pin_memory()
    ev2 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    # One graph per step also here when possible: [host-to-device copy of the step's inputs from a pinned
    # staging buffer] + [the five launches] + [device-to-host copy of the result into a pinned buffer].  The
    # host fills the staging buffer before every replay.
    from pqhsa_release_b200 import _lib

    e2e_graph = None
    hgather = None
    hstage = torch.empty_like(hin[0]).pin_memory()
    if runner.graph is not None and runner.exchange is not None:
        # sharded: the same graph form - [copy kernel for the inputs] + [the five launches, the last of which sends
        # the rows to all ranks] + [the receiving kernel, which unpacks every rank's rows straight into a pinned
        # host buffer mapped into the device's address space]
        hstage.copy_(hin[0])
        hgather = torch.zeros(2, *res_t.shape, dtype=res_t.dtype).pin_memory()
        pool.p.peer_gather = hgather.data_ptr()
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph):
            _lib.call("pqhsa_copy_small", runner.inbuf.data_ptr(), hstage.data_ptr(), hstage.numel() * hstage.element_size(),
                      torch.cuda.current_stream().cuda_stream)
            pool.decode_step_append(runner.q, runner.nk, runner.nv, encode=1, out=runner.out)
            runner.exchange.wait()
        pool.note_replayed(appends=-1, encodes=-1)  # the capture pass ran no kernels
    elif runner.graph is not None and world == 1:
        hstage.copy_(hin[0])
        e2e_graph = torch.cuda.CUDAGraph()
        # the result needs no copy node: the step's last kernel stores its output rows straight into the
        # pinned host buffer (mapped into the device's address space), 32 KB of posted writes over PCIe
        hview = hout.view(runner.out.shape)
        # ... and the inputs come in through a copy kernel that reads the pinned staging buffer over PCIe
        # (49 KB: quicker than a copy-engine node)
        with torch.cuda.graph(e2e_graph):
            _lib.call("pqhsa_copy_small", runner.inbuf.data_ptr(), hstage.data_ptr(), hstage.numel() * hstage.element_size(),
                      torch.cuda.current_stream().cuda_stream)
            pool.decode_step_append(runner.q, runner.nk, runner.nv, encode=1, out=hview)
        pool.note_replayed(appends=-1, encodes=-1)  # the capture pass ran no kernels

    def e2e_step(i):
        if e2e_graph is not None:
            torch.cuda.current_stream().synchronize()  # the previous replay has read the staging buffer
            hstage.copy_(hin[i % nq])
            flush_l2()
            ev2[i % K][0].record()
            e2e_graph.replay()
            pool.note_replayed(appends=1, encodes=1)
            runner.steps_done += 1
            ev2[i % K][1].record()
        else:
            flush_l2()
            ev2[i % K][0].record()
            runner.inbuf.copy_(hin[i % nq], non_blocking=True)  # q, new K rows, new V rows of the step
            runner.step()
            hout.copy_(runner.result(), non_blocking=True)
            ev2[i % K][1].record()

    for i in range(3):
        e2e_step(i)
    barrier()
    # once, outside the timed region: what arrived in the host buffer is the step's output (the same
    # query over the state the step left behind gives the same rows, up to summation order)
    if hgather is not None:
        # what the receiving kernel put into the host buffer = an NCCL all-gather of the ranks' rows
        torch.cuda.synchronize()
        hout.copy_(hgather[(runner.steps_done - 1) & 1])
        chk = torch.empty(world, *runner.out.shape, dtype=runner.out.dtype, device=device)
        torch.distributed.all_gather_into_tensor(chk.view(world * runner.out.shape[0], *runner.out.shape[1:]), runner.out)
        want = chk.reshape(-1, wl.head_dim).float().cpu()
    else:
        want = (runner.result() if world > 1 else pool.decode_step(runner.q)).reshape(-1, wl.head_dim).float().cpu()
    got = hout.clone().view(-1, wl.head_dim).float()
    if not bool(torch.isfinite(got).all()) or float((got - want).abs().max()) > 2e-2 * float(want.abs().max()):
        raise SystemExit("end-to-end check failed: the host buffer does not hold the step's output")
    for i in range(K):
        e2e_step(i)
    barrier()
    e2e_ms = sum(a.elapsed_time(b) for a, b in ev2)
    if hgather is not None:
        pool.p.peer_gather = runner.exchange.buf.data_ptr()  # back to the device buffer for what follows
    h2d = hin[0].numel() * hin[0].element_size()
    d2h = hout.numel() * hout.element_size()

    # ---- the latency floor of the step's launches: a graph of as many empty kernels, timed the same way ----
    n_launch = runner.launches_per_step + (1 if runner.exchange is not None else 0)
    floor_us = None
    if runner.graph is not None:
        stream = torch.cuda.current_stream().cuda_stream
        _lib.call("pqhsa_launch_empty", n_launch, stream)
        torch.cuda.synchronize()
        fg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(fg):
            _lib.call("pqhsa_launch_empty", n_launch, torch.cuda.current_stream().cuda_stream)
        nf = min(K, 50)
        evf = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nf)]
        for i in range(nf):
            flush_l2()
            evf[i][0].record(); fg.replay(); evf[i][1].record()
        torch.cuda.synchronize()
        floor_us = 1e3 * sum(a.elapsed_time(b) for a, b in evf) / nf

    # ---- end to end through the reference-facing object: GQASidecar.lean_append + forward, host buffers ----
    e2e_sidecar = None
    if world == 1 and not args.no_sidecar:
        e2e_sidecar = sidecar_e2e(wl, kv, qs, nks, nvs, n_start, min(K, 64), flush_l2, device)

    # ---- per-kernel durations inside a step --------------------------------
    # The five launches of a step are issued one by one with an event between them, right behind the L2
    # flush: the flush is still running while they are enqueued, so every event pair brackets exactly
    # one kernel as it runs inside the step (cold L2 at the start, what the step itself left in L2 after).
    from pqhsa_release_b200 import _lib

    stage_names = ["lut_build", "scan", "select", "attend", "merge"]
    reps = max(1, min(20, K))
    stage_ms = [0.0] * 5
    for r in range(reps):
        load_inputs(r)
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        flush_l2()
        evs[0].record()
        for sidx in range(5):
            pool.run_stage(sidx, runner.q, runner.out)
            evs[sidx + 1].record()
        torch.cuda.synchronize()
        for sidx in range(5):
            stage_ms[sidx] += evs[sidx].elapsed_time(evs[sidx + 1]) / reps
    barrier()

    # ---- aggregate ----------------------------------------------------------
    t = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    total_ms, e2e_ms = float(t[0]), float(t[1])
    keys_per_step = wl.batch * wl.kv_heads * n_start
    value = keys_per_step * K / (total_ms / 1e3)
    e2e_value = keys_per_step * K / (e2e_ms / 1e3)
    peak, peak_kind = measured_peaks()
    step_bytes = wl.algorithmic_bytes() + wl.batch * wl.kv_heads * (2 * wl.head_dim * 2 + 8)
    hl = wl.kv_heads // world
    e = 4 if wl.dtype == torch.float32 else 2
    f_rows = wl.context - wl.retrieval_len()
    # the attend kernel's algorithmic bytes: K selected + F sink/local K and V rows (sink/local rows once per
    # KV head) and the value means of the background
    attend_bytes = wl.batch * (hl * wl.group * wl.topk() + hl * f_rows) * 2 * wl.head_dim * e \
        + wl.batch * hl * wl.num_lists * wl.head_dim * e
    # dram__bytes_read.sum + dram__bytes_write.sum of one attend_kernel launch, from the committed ncu capture summary of this
    # workload under profiles/ (one GPU); no capture exists for other shapes
    traffic = profiled_traffic("attend_kernel") if (wl.name.startswith("c2") and world == 1 and not (args.context or args.batch)) else None
    attend_s = stage_ms[3] / 1e3
    achieved = attend_bytes / attend_s / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": total_ms / K, "us_per_layer_step": 1e3 * total_ms / K, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if wl.dtype == torch.bfloat16 else str(wl.dtype),
        "data": "synthetic",
        "config": {
            "workload": wl.name, "batch": wl.batch, "kv_heads": wl.kv_heads, "group": wl.group,
            "context": wl.context, "indexed_keys_per_stream": n_start, "topk": wl.topk(), "lists": wl.num_lists,
            "kv_layout": "contiguous", "index_update": "incremental, 1 key per step",
            "parallelism": f"kv-head shard x{world}",
            "exchange": "none" if world == 1 else ("flagged-word peer stores from the combine kernel + receiving kernel" if runner.exchange is not None
                                                   else "nccl all-gather"), "l2": f"flushed between timed steps ({args.flush} of 256 MiB)",
            "cuda_graph": not args.no_graph,
        },
        "step_roofline": {"algorithmic_bytes": step_bytes, "achieved_gbs": step_bytes / world / (total_ms / K / 1e3) / 1e9,
                          "peak_gbs": peak, "frac": step_bytes / world / (total_ms / K / 1e3) / 1e9 / peak,
                          "of": peak_kind},
        "roofline": {"kernel": "attend_kernel", "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": traffic, "of": peak_kind,
                     "algorithmic_bytes_per_launch": attend_bytes},
        "stages_us": {n: round(1e3 * m, 2) for n, m in zip(stage_names, stage_ms)},
        "e2e": {"value": e2e_value, "unit": UNIT, "us_per_layer_step": 1e3 * e2e_ms / K,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": n_launch * K,
        "launch_floor_us": floor_us,  # a CUDA graph of as many empty kernels as the step has launches, timed the same way
        "clocks": clocks,
        "wall_s_timed_region": wall, "setup_s": setup_s,
    }
    if e2e_sidecar is not None:
        line["e2e_sidecar"] = e2e_sidecar
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_reference(wl, budget_s=20.0, steps=20, warmup=3)["cpu_baseline"]
    if rank == 0:
        if args.stages:
            print(json.dumps(line["stages_us"]), file=sys.stderr)
        print(json.dumps(line))
    if world > 1:
        # Leave without tearing NCCL down: destroying a communicator whose kernels sit in a live CUDA
        # graph can block for ever.  Every rank has printed / finished once the barrier returns.
        sys.stdout.flush()
        sys.stderr.flush()
        runner.graph = None
        torch.cuda.synchronize()
        torch.distributed.barrier()
        torch.cuda.synchronize()
        os._exit(0)


# --------------------------------------------------------------------------
# c3: the paged plugin path (vLLM page layout, ragged batch, one key appended and encoded per step)
# --------------------------------------------------------------------------
def run_paged_plugin(args):
    """Workloads c3 and c4 through the plugin's own entry, ``pq_or_dense_forward``.

    c3: 16 requests with contexts drawn uniformly from [8192, 65536], 16-token pages in vLLM's
    [blocks, Hkv, block_size, 2D] layout behind a randomly permuted block table; every decode step stores one
    K/V row per head in the pages (vLLM's own cache write, outside the timed region as in the reference's
    attention segment) and the hook appends it, encodes the key that leaves the local window and attends -
    one fused library call per layer-step.  One layer, one GPU.

    c4: Llama-3-70B attention shape (8 KV heads, GQA 8), 80 layers with independent synthetic KV, context
    262144, batch 8, the KV heads sharded over the ranks as vLLM's tensor parallelism does (one head per GPU on
    8 GPUs; every rank holds its heads' pages and index and runs this same path - the attention outputs stay
    sharded, as in vLLM, where the row-parallel output projection follows).  A step = all 80 layers; the
    production index policy (deferred, flush every 256 tokens).  ``value`` counts the keys of all layers and ranks."""
    from types import SimpleNamespace as NS

    from pqhsa_release_b200.pq_hsa_vllm import runtime

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    wl = workloads.WORKLOADS[args.workload]
    is_c4 = args.workload == "c4"
    if not is_c4 and world > 1:
        raise SystemExit("workload c3 is measured on one GPU")
    if wl.kv_heads % world:
        raise SystemExit(f"{wl.kv_heads} KV heads do not shard over {world} ranks")
    B = args.batch or wl.batch
    layers = (args.layers or 80) if is_c4 else 1
    K, W = args.steps, max(args.warmup, 3)
    Hkv, G, D, bs = wl.kv_heads // world, wl.group, wl.head_dim, wl.block_size
    Hq = Hkv * G
    g = torch.Generator().manual_seed(33)
    if is_c4:
        ctxs = [args.context or wl.context] * B
    else:
        ctxs = [int(x) for x in torch.randint(8192, (args.context or wl.context) + 1, (B,), generator=g)]
    need_gb = layers * sum(ctxs) * Hkv * 2 * D * 2 / 2 ** 30
    if need_gb > 150:
        raise SystemExit(f"{need_gb:.0f} GiB of KV pages per GPU do not fit: use more ranks (--gpus) or fewer --layers")
    grow = W + 2 * K + 32   # tokens a request gains over the whole run: warm-up, the timed steps, the end-to-end steps
    blocks_of = [(c + grow + bs - 1) // bs for c in ctxs]
    max_blocks = max(blocks_of)
    nblk = sum(blocks_of) + 16
    perm = torch.randperm(nblk, generator=g)
    table = torch.zeros(B, max_blocks, dtype=torch.int32)
    at = 0
    for b, nb in enumerate(blocks_of):
        table[b, :nb] = perm[at : at + nb].to(torch.int32)
        at += nb
    table = table.to(device)
    t0 = time.time()
    caches, q_layers = [], []
    for layer_i in range(layers):
        kv_cache = torch.zeros(nblk, Hkv, bs, 2 * D, dtype=wl.dtype, device=device)
        qs = []
        for b, c in enumerate(ctxs):
            k, v = workloads.mixture_kv(300_000 + 1000 * layer_i + 10 * b + rank, Hkv, c, dtype=wl.dtype, device=device)
            t = torch.arange(c, device=device)
            blk, off = table[b, t // bs].long(), t % bs
            kv_cache[blk, :, off, :D] = k.permute(1, 0, 2)
            kv_cache[blk, :, off, D:] = v.permute(1, 0, 2)
            qs.append(workloads.planted_queries(7_000 + b + 31 * layer_i, k, G))
            del k, v
        caches.append(kv_cache)
        q_layers.append(torch.stack(qs).contiguous())  # [B, Hq, D]
    env = {"PQ_HSA_BATCH": "1", "PQ_HSA_TOP_FRAC": str(wl.top_fraction), "PQ_HSA_NUM_LISTS": str(wl.num_lists),
           "PQ_HSA_MAX_REQUESTS": str(B), "PQ_HSA_MAX_CONTEXT": str(max_blocks * bs), "PQ_HSA_ENABLE": "1",
           "PQ_HSA_SINK": str(wl.sink_tokens), "PQ_HSA_LOCAL": str(wl.local_window), "PQ_HSA_PREFIX_CACHE": "0"}
    env.update({"PQ_HSA_UPD_STRATEGY": "deferred", "PQ_HSA_UPD_INTERVAL": "256", "PQ_HSA_FLUSH_INTERVAL": "256"} if is_c4 else
               {"PQ_HSA_UPD_STRATEGY": "incremental", "PQ_HSA_UPD_INTERVAL": "1"})
    os.environ.update(env)
    runtime.reset()
    runner = NS(input_batch=NS(req_ids=[f"req{b}" for b in range(B)]), requests={})
    impl = NS(scale=1.0 / math.sqrt(D), num_heads=Hq, num_kv_heads=Hkv, kv_cache_dtype="auto")
    layer_objs = [object() for _ in range(layers)]
    lens = list(ctxs)

    def dense(*a, **k):
        raise SystemExit("the step fell through to the dense path: " + str(runtime.rejects()))

    nq = 4
    gd = torch.Generator(device=device).manual_seed(5 + rank)
    rows = [(torch.randn(B, Hkv, D, generator=gd, device=device).to(wl.dtype), torch.randn(B, Hkv, D, generator=gd, device=device).to(wl.dtype))
            for _ in range(nq)]
    out = torch.zeros(layers, B, Hq * D, dtype=wl.dtype, device=device)
    hq = torch.stack(q_layers).cpu().pin_memory()            # [layers, B, Hq, D]: the step's queries on the host
    q_dev = torch.zeros(layers, B, Hq, D, dtype=wl.dtype, device=device)
    hout = torch.empty(layers, B, Hq * D, dtype=wl.dtype).pin_memory()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    flush_rd = torch.zeros(64 << 20, dtype=torch.int32, device=device)
    bidx = torch.arange(B, device=device)

    def vllm_cache_write(i):
        """What vLLM does before the attention forwards: the step's K/V rows go into every layer's pages."""
        nk, nv = rows[i % nq]
        pos = torch.tensor(lens, device=device)
        blk, off = table[bidx, pos // bs].long(), pos % bs
        for kv_cache in caches:
            kv_cache[blk, :, off, :D] = nk
            kv_cache[blk, :, off, D:] = nv
        for b in range(B):
            lens[b] += 1
        return nk, nv

    def metadata():
        t = torch.tensor(lens, dtype=torch.int32)
        return NS(use_cascade=False, max_query_len=1, num_actual_tokens=B, seq_lens=t, seq_lens_cpu=t, max_seq_len=max(lens),
                  block_table=table, slot_mapping=None, _pq_runner=runner)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def step(i, e2e=False, ev=None):
        nk, nv = vllm_cache_write(i)
        md = metadata()
        flush.zero_(); flush_rd.sum()
        if ev is not None:
            ev[0].record()
        if e2e:
            q_dev.copy_(hq, non_blocking=True)
        for li in range(layers):
            q = q_dev[li] if e2e else q_layers[li]
            runtime.pq_or_dense_forward(dense, impl, layer_objs[li], q, nk, nv, caches[li], md, output=out[li])
        if e2e:
            hout.copy_(out, non_blocking=True)
        if ev is not None:
            ev[1].record()

    step(0)                     # builds every layer's and request's index
    barrier()
    setup_s = time.time() - t0
    for i in range(1, W):
        step(i)
    barrier()
    engines = [runtime._LAYERS[id(l)] for l in layer_objs]
    n_keys = sum(int((e.pool.h_sorted + e.pool.h_tail)[: B * Hkv].sum()) for e in engines)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    sampler.start()
    for i in range(K):
        step(W + i, ev=ev[i])
    barrier()
    clocks = sampler.stop()
    total_ms = sum(a.elapsed_time(b) for a, b in ev)
    ev2 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    for i in range(K):
        step(W + K + i, e2e=True, ev=ev2[i])
    barrier()
    e2e_ms = sum(a.elapsed_time(b) for a, b in ev2)
    if not bool(torch.isfinite(hout.float()).all()):
        raise SystemExit("end-to-end check failed: the host buffer holds non-finite values")
    assert runtime.STATS["builds"] == B * layers and runtime.STATS["dense_steps"] == 0, runtime.STATS
    # per-kernel durations of one layer-step, launched stage by stage behind the flush (first layer)
    import ctypes as C

    from pqhsa_release_b200 import _lib

    stage_names = ["lut_build", "scan", "select", "attend", "merge"]
    stage_ms = [0.0] * 5
    reps = min(10, K)
    pool = engines[0].pool
    launches = 5 + (1 if pool.layout.parts > 1 else 0)  # tables, scan, selection (one or two), attend, combine
    for r in range(reps):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        flush.zero_(); flush_rd.sum()
        evs[0].record()
        for sidx in range(5):
            pool.p.q, pool.p.out = q_layers[0].data_ptr(), out[0].data_ptr()
            _lib.call("pqhsa_run_stage", C.byref(pool.p), sidx, torch.cuda.current_stream().cuda_stream)
            evs[sidx + 1].record()
        torch.cuda.synchronize()
        for sidx in range(5):
            stage_ms[sidx] += evs[sidx].elapsed_time(evs[sidx + 1]) / reps
    t = torch.tensor([total_ms, e2e_ms, float(n_keys)], dtype=torch.float64, device=device)
    if world > 1:
        tm = t.clone()
        torch.distributed.all_reduce(tm, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.SUM)
        total_ms, e2e_ms, n_keys = float(tm[0]), float(tm[1]), int(t[2])
    peak, peak_kind = measured_peaks()
    mid = [c + W + K // 2 for c in ctxs]
    step_bytes = layers * (wl.algorithmic_bytes(contexts=mid) + (B * wl.kv_heads * (2 * D * 2 + 8) if not is_c4 else 0))
    e = 2
    attend_bytes = sum(Hq * wl.topk(c) * 2 * D * e + Hkv * (c - wl.retrieval_len(c)) * 2 * D * e + Hkv * wl.num_lists * D * e
                       for c in ctxs)
    achieved = attend_bytes / (stage_ms[3] / 1e3) / 1e9
    per_layer_us = 1e3 * total_ms / K / layers
    line = {
        "metric": METRIC, "value": n_keys * K / (total_ms / 1e3), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": total_ms / K, "us_per_layer_step": per_layer_us, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wl.name, "batch": B, "kv_heads": wl.kv_heads, "group": G, "layers": layers,
                   "contexts": ctxs if not is_c4 else ctxs[0], "indexed_keys_all_layers_and_ranks": n_keys, "lists": wl.num_lists,
                   "kv_layout": "paged: vLLM [blocks, Hkv, 16, 2D] pages, permuted block table",
                   "index_update": "deferred, flush every 256 tokens" if is_c4 else "incremental, 1 key per request-head and step",
                   "entry": f"pq_hsa_vllm runtime.pq_or_dense_forward (eager, {launches} launches per layer-step)",
                   "parallelism": f"kv-head shard x{world}, attention outputs stay sharded (vLLM tensor parallelism)",
                   "l2": "flushed between timed steps (write+read of 256 MiB)", "cuda_graph": False},
        "step_roofline": {"algorithmic_bytes": step_bytes, "achieved_gbs": step_bytes / world / (total_ms / K / 1e3) / 1e9,
                          "peak_gbs": peak, "frac": step_bytes / world / (total_ms / K / 1e3) / 1e9 / peak, "of": peak_kind},
        "roofline": {"kernel": "attend_kernel", "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "of": peak_kind, "algorithmic_bytes_per_launch": attend_bytes},
        "stages_us": {n: round(1e3 * m, 2) for n, m in zip(stage_names, stage_ms)},
        "e2e": {"value": n_keys * K / (e2e_ms / 1e3), "unit": UNIT, "us_per_layer_step": 1e3 * e2e_ms / K / layers,
                "h2d_bytes_per_step": hq.numel() * 2, "d2h_bytes_per_step": hout.numel() * 2},
        "gpu_launches": launches * K * layers, "clocks": clocks, "setup_s": setup_s, "runtime_stats": dict(runtime.STATS),
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from dataclasses import replace

        line["cpu_baseline"] = cpu_reference(replace(wl, batch=B, context=int(sum(ctxs) / B)), budget_s=20.0, steps=3, warmup=1)["cpu_baseline"]
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        sys.stdout.flush()
        torch.cuda.synchronize()
        torch.distributed.barrier()
        os._exit(0)


# --------------------------------------------------------------------------
# reference arm: the CPU port of the reference's torch path (oracle/)
# --------------------------------------------------------------------------
def cpu_reference(wl, budget_s, steps, warmup):
    """Time the restated reference path (IVFPQSparseAttention.forward_many per stream,
    fp32, as benchmarks/vllm_backend/gqa_sidecar.py drives it) on the host cores for a
    bounded sample of the workload's streams; extrapolate to all streams."""
    from oracle.pqhsa_oracle import OracleAttentionConfig, OracleIndexConfig, OracleStream

    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except Exception:
        pass
    torch.set_num_threads(cores)
    n_streams = wl.batch * wl.kv_heads
    sample = []
    t_build = time.perf_counter()
    # at most four full-context streams: the index build dominates the sample's cost
    for i in range(min(4, n_streams)):
        k, v = workloads.mixture_kv(100_000 * 0 + i, 1, wl.context, dtype=wl.dtype)
        st = OracleStream(
            OracleIndexConfig(num_lists=wl.num_lists),
            OracleAttentionConfig(sink_tokens=wl.sink_tokens, local_window=wl.local_window,
                                  retrieval_top_fraction=wl.top_fraction, index_update_interval=1,
                                  index_update_strategy="incremental"),
        ).build_cache(k[0].float(), v[0].float())
        q = workloads.planted_queries(7_000 + i, k, wl.group).float()
        sample.append((st, q))
        if time.perf_counter() - t_build > budget_s:
            break
    build_s = time.perf_counter() - t_build
    g = torch.Generator().manual_seed(1)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for st, q in sample:
            st.append(torch.randn(wl.head_dim, generator=g), torch.randn(wl.head_dim, generator=g))
            st.forward_many(q)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    per_stream = sorted(times)[len(times) // 2] / len(sample)
    step_s = per_stream * n_streams
    n_keys = wl.batch * wl.kv_heads * wl.retrieval_len()
    value = n_keys / step_s
    desc = (f"{len(sample)} of {n_streams} streams at full context ({wl.context}), {steps} steps after {warmup} "
            f"warm-up, per-stream median x {n_streams} (extrapolated); index build {build_s:.1f} s not included")
    return {
        "value": value, "ms_per_step": 1e3 * step_s,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc,
                         "us_per_layer_step": 1e6 * step_s},
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = workloads.WORKLOADS[args.workload]
    if args.context or args.batch:
        from dataclasses import replace

        wl = replace(wl, context=args.context or wl.context, batch=args.batch or wl.batch)
    # a step of this arm is the sample's four streams (about 13 ms each at c2): the driver's step count is
    # honoured up to 200, never fewer than 20 after at least 3 warm-up steps
    steps, warmup = max(20, min(args.steps, 200)), max(3, min(args.warmup, 10))
    r = cpu_reference(wl, budget_s=60.0, steps=steps, warmup=warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl.name, "batch": wl.batch, "kv_heads": wl.kv_heads, "group": wl.group,
                   "context": wl.context, "note": "CPU port of the reference torch path, host cores only"},
        "cpu_baseline": r["cpu_baseline"],
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_encode_bulk(args):
    """``--workload encode_bulk``: the bulk encode kernel (the pass that ends an index build or a codebook-moving
    refresh: every key assigned to its nearest list and PQ-encoded) on seeded synthetic keys of the c2 index size,
    and whole ``build_index_batch`` / ``online_refresh_batch`` calls around it.  One JSON line of its own."""
    from pqhsa_release_b200.config import paper_index_config
    from pqhsa_release_b200.index_build import build_index_batch, encode_bulk, online_refresh_batch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    streams, keys, lists, dt = (args.batch or 4) * 8, (args.context or 131072) - 132, 512, torch.bfloat16
    iters = max(3, min(args.steps, 20))
    gen = torch.Generator(device="cuda").manual_seed(0)
    k = torch.randn(streams, keys, 128, device="cuda", generator=gen).to(dt)
    coarse = torch.nn.functional.normalize(torch.randn(streams, lists, 128, device="cuda", generator=gen), dim=-1).to(dt)
    books = (0.1 * torch.randn(streams, 8, 16, 16, device="cuda", generator=gen)).to(dt)
    for _ in range(max(args.warmup, 1)):
        encode_bulk(k, coarse, books)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(iters):
        encode_bulk(k, coarse, books)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / iters
    del k, coarse, books
    cfg = paper_index_config(num_lists=lists)
    kk = torch.randn(streams, keys + 256, 128, device="cuda").to(dt)
    vv = torch.randn(streams, keys + 256, 128, device="cuda").to(dt)
    def timed(fn):
        torch.cuda.synchronize()
        t = time.perf_counter()
        res = fn()
        torch.cuda.synchronize()
        return res, (time.perf_counter() - t) * 1e3

    # every call three times: the first one also pays for the device allocations of its temporaries (torch's
    # allocator keeps them afterwards); the median is reported, all three are listed
    torch.cuda.reset_peak_memory_stats()
    base_gib = torch.cuda.memory_allocated() / 2 ** 30
    build_calls = []
    for _ in range(3):
        built, t = timed(lambda: build_index_batch(kk[:, :keys], vv[:, :keys], cfg))
        build_calls.append(t)
    peak_gib = torch.cuda.max_memory_allocated() / 2 ** 30 - base_gib
    cur = [{"coarse": b.coarse_centroids, "codebooks": b.codebooks} for b in built]
    refresh_calls = [timed(lambda: online_refresh_batch(kk, vv, cur, 256, cfg))[1] for _ in range(3)]
    build_ms, refresh_ms = sorted(build_calls)[1], sorted(refresh_calls)[1]
    pairs = streams * keys * lists * 128
    fp32_issue = 148 * 128 * 1.965e9 / 2  # subtract + fma per pair: nominal, there is no measured fp32 peak
    print(json.dumps({
        "metric": "index_encode_keys_per_s", "value": streams * keys / (ms / 1e3), "unit": "keys/s", "n_gpus": 1,
        "steps": iters, "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "encode_bulk: index build / refresh pass at the c2 index size", "streams": streams,
                   "keys_per_stream": keys, "lists": lists, "element": "bf16"},
        "roofline": {"bound": "fp32 issue (nominal)", "achieved": pairs / (ms / 1e3) / 1e12, "peak": fp32_issue / 1e12,
                     "unit": "T subtract-fma pairs/s", "frac": pairs / (ms / 1e3) / fp32_issue, "traffic": None},
        "build_index_batch_ms": build_ms, "build_temporaries_gib": peak_gib, "online_refresh_batch_ms": refresh_ms,
        "calls_ms": {"build_index_batch": build_calls, "online_refresh_batch": refresh_calls},
        "note": "whole calls, wall clock around a device synchronise; the median of three calls each",
    }))


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    elif a.workload in ("c3", "c4"):
        run_paged_plugin(a)
    elif a.workload == "encode_bulk":
        run_encode_bulk(a)
    else:
        run_b200(a)
