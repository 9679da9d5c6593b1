#!/usr/bin/env python3
"""Benchmark of the routed selection-and-reduction path: ctx-512, K=8 stateful decode.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode position for a batch of sequences (one pass of the hot path:
packed projection -> cache append / router update -> per layer select -> relation hidden ->
second MLP layer -> norm-reduce -> heads).  Workload = the 6-layer ctx-512 configuration: 6 relation layers,
d_model 512, vocab 16000 + 256 boundary ids, context 512 (448-token prefix, then generated
positions), block 32, local window 64, 2 remote blocks, 1 anchor, K = 8, bf16, batch 8 per
GPU.  Token ids are bounded Zipf(s = 1.1) over the vocabulary, boundary ids uniform; weights
are seeded random init.  These synthetic inputs stand in for the reference's private
checkpoint and validation text.

Prints ONE JSON line (rank 0).  ``value`` = tokens/s over all GPUs with every input resident
in HBM, each step's CUDA-event time summed, the L2 flushed between steps.  ``e2e`` = the same
metric through the host API: token ids copied from pinned host memory and the greedy next
token read back every step.  ``roofline`` describes the library kernel with the largest
share of a step; ``cpu_baseline`` is the CPU port of the same step timed on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "relation-lm_b200"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import torch  # noqa: E402

PREFIX = 448
METRIC = "relation decode tokens/s at ctx512 K=8"
UNIT = "tokens/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one relation_select_kernel launch at 256 rows of the
# 12-layer decode shape (ncu capture summarised under profiles/), and its ratio to the algorithmic bytes
NCU_SELECT_TRAFFIC_ROWS256 = 21_464_576
NCU_SELECT_TRAFFIC_RATIO = 21_464_576 / 21_325_824
CPU_SAMPLE_BATCH = 8   # the CPU arm keeps fp32 caches on the host: it decodes at most this many sequences


def log(message: str) -> None:
    print(f"[bench {time.strftime('%H:%M:%S')}] {message}", file=sys.stderr, flush=True)


def zipf_tokens(batch: int, length: int, vocab: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    weights = torch.arange(1, vocab + 1, dtype=torch.float64).pow(-1.1)
    return torch.multinomial(weights / weights.sum(), batch * length, replacement=True,
                             generator=g).view(batch, length)


def make_model(workload: str):
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM

    if workload == "cfg5":
        cfg = RoutedRelationConfig(d_model=768, layers=12, max_context=2048, block_size=64,
                                   local_window=128, top_blocks=2)
        seed = 1005
    else:
        cfg = RoutedRelationConfig()
        seed = 1002
    return RoutedRelationLM(cfg, seed=seed), seed


# ---------------------------------------------------------------------------- clocks


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.samples: list[list[str]] = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            deadline = time.time() + 3.0               # nvidia-smi needs a moment before its first line
            while not self.samples and time.time() < deadline:
                time.sleep(0.01)
            self.samples.clear()                        # keep only what is sampled from here on
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 7:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[3:7]) if v == "Active"})
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": float(self.samples[0][1]) if self.samples else None,
                "samples": len(self.samples), "reasons": reasons}


# ---------------------------------------------------------------------------- CPU arm


def cpu_decode_rate(workload: str, batch: int, steps: int, warmup: int, threads: int):
    """The CPU port of the decode step on the host cores, from a synthetic state at the end
    of the prefix (cache contents do not change the work done)."""
    import oracle
    from oracle.decode_port import OracleDecoder

    threads = threads or (os.cpu_count() or 1)
    torch.set_num_threads(threads)
    oracle.set_threads(threads)
    model, seed = make_model(workload)
    cfg = model.config
    prefix = cfg.max_context - 64
    dec = OracleDecoder(model, batch, torch.float32)
    g = torch.Generator().manual_seed(seed)
    for t in (dec.anchor_keys, dec.partner_keys, dec.operand_cache, dec.partner_anchor_cache,
              dec.expanded_cache, *dec.router_caches):
        t[:, :, :prefix].normal_(generator=g)
    for i, s in enumerate(dec.router_stats):
        s[:, :, :prefix // cfg.block_size].normal_(generator=g)
        if i % 2 == 1:
            s.abs_()
    dec.position = prefix
    tokens = zipf_tokens(batch, warmup + steps, cfg.vocab_size, seed)
    bounds = torch.randint(0, cfg.boundary_vocab_size, (batch, warmup + steps), generator=g)
    for i in range(warmup):
        dec.step(tokens[:, i], bounds[:, i])
    start = time.perf_counter()
    for i in range(warmup, warmup + steps):
        if dec.position >= cfg.max_context:
            dec.position = prefix
        dec.step(tokens[:, i], bounds[:, i])
    elapsed = time.perf_counter() - start
    return batch * steps / elapsed, elapsed, threads


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    cpu_batch = min(args.batch, CPU_SAMPLE_BATCH)
    value, elapsed, threads = cpu_decode_rate(args.workload, cpu_batch, steps, args.warmup, 0)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": elapsed / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(args.workload, args.batch, 1),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{steps} decode positions of {cpu_batch} of the {args.batch} sequences from a synthetic "
                                   "end-of-prefix state, CPU port of the step (C oracle + fp32 torch matmuls)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference ships no CPU-runnable sparse decode (its kernels are Triton-only and its "
                "decode driver is not public); this arm times the CPU restatement of the same step",
    }
    print(json.dumps(line), flush=True)


def workload_config(workload: str, batch: int, n_gpus: int) -> dict:
    if workload == "cfg5":
        return {"workload": "cfg5 batch-sharded stateful decode: 12 layers, d_model 768, ctx 2048, "
                            "block 64, window 128, 2 remote blocks, 1 anchor, K=8",
                "batch_per_gpu": batch, "global_batch": batch * n_gpus, "l2": "flushed between steps"}
    return {"workload": "cfg2 routed stateful decode: 6 layers, d_model 512, ctx 512 (448 prefix), "
                        "block 32, window 64, 2 remote blocks, 1 anchor, K=8",
            "batch_per_gpu": batch, "global_batch": batch * n_gpus, "l2": "flushed between steps"}


# ---------------------------------------------------------------------------- rank sharding


def rank_inputs(cfg, seed: int, batch: int, rank: int):
    """The token / boundary ids of this rank's sequences: every rank decodes its own `batch`
    sequences (weak scaling), drawn from a rank-specific seed."""
    tokens = zipf_tokens(batch, cfg.max_context, cfg.vocab_size, seed + rank)
    bounds = torch.randint(0, cfg.boundary_vocab_size, (batch, cfg.max_context),
                           generator=torch.Generator().manual_seed(seed + 77 + rank))
    return tokens, bounds


def max_over_ranks(values, world: int, device) -> list[float]:
    """Element-wise maximum of per-rank timings (the slowest rank defines the job's time)."""
    times = torch.tensor(list(values), device=device, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    return [float(v) for v in times.tolist()]


def job_rate(world: int, batch_per_rank: int, steps: int, max_ms: float) -> float:
    """Whole-job tokens/s: the positions all ranks decoded divided by the slowest rank's time."""
    return world * batch_per_rank * steps / (max_ms / 1e3)


# ---------------------------------------------------------------------------- GPU arm


def kernel_table(dec, graph_iters: int = 20):
    """Average launch duration of each library kernel on the decoder's own state, captured in
    CUDA graphs (one launch per layer per graph, so consecutive launches touch different
    caches), with the algorithmic bytes of the per-row formulas (tensors a launch must read or write, once)."""
    from relation_lm.kernels.packed_projection import packed_projection
    from relation_lm.kernels.relation_reduce import (expanded_cache_append, relation_hidden_cache_update_out,
                                                     relation_hidden_cached_out, relation_norm_reduce_residual)
    from relation_lm.kernels.relation_select import relation_select_packed
    from relation_lm.kernels.router_cache import sparse_cache_append

    cfg, w, B = dec.config, dec.w, dec.batch
    stacked = getattr(dec, "stacked_expand", False)
    L, K, H, R, d = cfg.layers, cfg.k_max, cfg.hidden_dim, cfg.relation_dim, cfg.d_model
    dev = dec.device
    e = dec.anchor_keys.element_size()
    pos = torch.tensor(cfg.max_context - 1, device=dev, dtype=torch.int64)
    packed = torch.randn(B, L * (384 + R), device=dev).to(dec.dtype)
    q = torch.randn(B, 256, device=dev).to(dec.dtype)
    anchor = torch.randint(0, cfg.max_context, (B,), device=dev, dtype=torch.int32)
    partner = torch.randint(0, cfg.max_context, (B, K), device=dev, dtype=torch.int32)
    scores = torch.randn(B, K, device=dev)
    raw = torch.randn(L, B, K, d, device=dev).to(dec.dtype)
    hidden_out = torch.empty(B, K, H, device=dev, dtype=dec.dtype)
    residual = torch.randn(B, d, device=dev)

    def select(l):
        relation_select_packed(q[:, 0:64], dec.anchor_keys[l], q[:, 64:128], dec.router_stats[0][l],
                               dec.router_stats[1][l], w["anchor_gamma"][l], w["anchor_bias"][l],
                               q[:, 128:256], dec.partner_anchor_cache[l], dec.partner_keys[l],
                               dec.router_stats[2][l], dec.router_stats[3][l], w["partner_gamma"][l],
                               w["partner_bias"][l], pos, cfg.local_window, cfg.top_blocks, K, cfg.strict_valid)

    def hidden(l):
        if stacked:
            relation_hidden_cached_out(hidden_out, dec.expanded_cache[l], dec.operand_cache[l], anchor,
                                       partner, w["product_weight"][l])
        else:
            relation_hidden_cache_update_out(hidden_out, dec.expanded_cache[l], dec.operand_cache[l], anchor,
                                             partner, w["anchor_weight"][l], w["partner_weight"][l],
                                             w["product_weight"][l], w["first_bias"][l], pos)

    def expand(_):
        expanded_cache_append(dec.expanded_cache, dec.operand_cache, w["anchor_weight"], w["partner_weight"],
                              w["first_bias"], pos)

    def reduce(l):
        relation_norm_reduce_residual(raw[l], scores, w["relation_norm_w"][l], w["relation_norm_b"][l], pos,
                                      cfg.norm_eps, residual, w["mix"][l])

    normalized = torch.randn(B, d, device=dev).to(dec.dtype)
    fused_query = getattr(dec, "fused_query", False)
    projected = torch.empty(B, 256, device=dev, dtype=dec.dtype)

    def reduce_project(l):
        from relation_lm.kernels.relation_reduce import relation_norm_reduce_residual_norm_project
        relation_norm_reduce_residual_norm_project(
            raw[l], scores, w["relation_norm_w"][l], w["relation_norm_b"][l], pos, cfg.norm_eps, residual,
            w["mix"][l], w["input_norm_w"][l], w["input_norm_b"][l], cfg.norm_eps, normalized,
            w["w_query"][l], projected)

    def query(l):
        packed_projection(normalized, w["w_query"][l])

    def append(_):
        sparse_cache_append(packed, dec.anchor_keys, dec.partner_keys, dec.operand_cache,
                            dec.partner_anchor_cache, *dec.router_caches, *dec.router_stats,
                            w["anchor_conv_weight"], w["partner_conv_weight"], pos, cfg.block_size)

    cand = cfg.local_window + cfg.top_blocks * cfg.block_size
    nb = cfg.max_context // cfg.block_size
    bytes_per_launch = {
        "relation_select_kernel": B * (e * (4 * nb * 64 + 2 * cand * 64 + 64 + 64 + 128 + 128) + 2 * (4 + 64) * 4 + 8 + 8 * K),
        "relation_hidden_kernel": B * (e * ((1 + K) * H + (1 + K) * R) + 8 + 4 * K + e * K * H) + e * H * R
                                  + (0 if stacked else e * 2 * H * R + B * e * (R + 2 * H)),
        "expanded_row_update_kernel(all layers)": L * (e * 2 * H * R + B * e * (R + 2 * H)),
        "relation_norm_reduce_kernel": B * (e * K * d + 4 * K + 4 * d + 8 * d) + 4 * 3 * d,
        "packed_projection_kernel(query)": e * (B * d + 256 * d + B * 256),
        "relation_norm_reduce_project_kernel": B * (e * K * d + 4 * K + 4 * d + 8 * d) + 4 * 3 * d
                                               + e * (B * d + 256 * d + B * 256),
        "router_cache_update_kernel(all layers)": L * B * (e * 64 * (2 + 4 + 4 + 2 * cfg.block_size + 4) + 2 * 64 * 4 + 2 * e * (256 + R)),
    }
    table = {}
    # (kernel, launcher, launches per timing graph, launches per decode step): with the query
    # projection inside norm-reduce only layer 0 projects separately and only the last layer's
    # norm-reduce runs without a projection
    for name, fn, per_graph, per_step in (
            ("relation_select_kernel", select, L, L),
            ("relation_hidden_kernel", hidden, L, L),
            ("relation_norm_reduce_kernel", reduce, L, 1 if fused_query else L),
            ("relation_norm_reduce_project_kernel", reduce_project, L, L - 1),
            ("packed_projection_kernel(query)", query, L, 1 if fused_query else L),
            ("router_cache_update_kernel(all layers)", append, 1, 1),
            ("expanded_row_update_kernel(all layers)", expand, 1, 1)):
        if name.startswith("expanded_row_update") and not stacked:
            continue
        if name == "relation_norm_reduce_project_kernel" and not fused_query:
            continue
        for l in range(per_graph):
            fn(l)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for l in range(per_graph):
                    fn(l)
        torch.cuda.synchronize()
        for _ in range(3):
            graph.replay()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(graph_iters):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(end) * 1e3 / (graph_iters * per_graph)
        launches_per_step = per_step
        table[name] = {"us_per_launch": us, "launches_per_step": launches_per_step,
                       "us_per_step": us * launches_per_step, "bytes_per_launch": bytes_per_launch[name],
                       "gb_per_s": bytes_per_launch[name] / us / 1e3}
    return table


def select_rows256(device, graph_iters: int = 10):
    """The selector at the row count where bandwidth starts to matter: 256 rows of the 12-layer
    decode shape (ctx 2048, block 64, window 128, 2 remote blocks, K 8, bf16), three cache sets of
    268 MB so that consecutive launches miss L2, timed inside a captured graph."""
    from relation_lm.kernels.relation_select import relation_select_packed

    B, T, bs, L, TOP, K = 256, 2048, 64, 128, 2, 8
    nb, sets = T // bs, 3
    rn = lambda *shape: torch.randn(*shape, device=device).bfloat16()  # noqa: E731
    S = [(rn(B, T, 64), rn(B, T, 64), rn(B, T, 128), rn(B, nb, 4, 16), rn(B, nb, 4, 16).abs(),
          rn(B, nb, 4, 16), rn(B, nb, 4, 16).abs()) for _ in range(sets)]
    q, g, bias = rn(B, 256), torch.randn(4, device=device), torch.randn(4, 16, device=device)
    pos = torch.tensor(T - 1, device=device)

    def launch(i):
        ak, pk, pac, am, as_, pm, ps = S[i]
        relation_select_packed(q[:, :64], ak, q[:, 64:128], am, as_, g, bias, q[:, 128:], pac, pk, pm, ps,
                               g, bias, pos, L, TOP, K, False)

    launch(0)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for i in range(sets):
                launch(i)
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(graph_iters):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(end) * 1e3 / (graph_iters * sets)
    cand = L + TOP * bs
    nbytes = B * (2 * (4 * nb * 64 + 2 * cand * 64 + 64 + 64 + 128 + 128) + 2 * (4 + 64) * 4 + 8 + 8 * K)
    return {"kernel": "relation_select_kernel", "rows": B, "us_per_launch": us, "bytes_per_launch": nbytes,
            "gb_per_s": nbytes / us / 1e3}


def run_ours(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the library has no CPU fallback)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        # NCCL announces its version on stdout at the first collective; keep stdout for the JSON line
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    from relation_lm.inference.stateful_decode import StatefulDecoder
    from relation_lm.kernels import _abi

    model, seed = make_model(args.workload)
    cfg = model.config
    B, T = args.batch, cfg.max_context
    prefix = T - 64 if args.prefix is None else args.prefix
    dec = StatefulDecoder(model, B, device, torch.bfloat16)
    tokens, bounds = rank_inputs(cfg, seed, B, rank)
    tokens, bounds = tokens.to(device), bounds.to(device)

    log(f"state allocated: {dec.state_bytes() / 1e9:.1f} GB")
    launches_before = _abi.launch_count()
    dec.step_greedy(tokens[:, 0], bounds[:, 0])          # what the captured graph replays
    kernels_per_step = _abi.launch_count() - launches_before
    dec.reset()
    dec.capture()
    # prefix: PREFIX positions through the captured step
    for t in range(prefix):
        dec.static_tokens.copy_(tokens[:, t])
        dec.static_boundaries.copy_(bounds[:, t])
        dec.replay()
    torch.cuda.synchronize()
    log(f"prefix of {prefix} positions done")
    assert int(dec.position.item()) == prefix
    assert _abi.read_status() == 0, "a kernel reported a device-side error during the prefix"

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)

    def run_steps(count: int, timed: bool):
        events = []
        for i in range(count):
            t = prefix + (int(run_steps.done) % 64)
            if t == prefix and run_steps.done:
                dec.position.fill_(prefix)
            dec.static_tokens.copy_(tokens[:, t])
            dec.static_boundaries.copy_(bounds[:, t])
            flush.zero_()
            if timed:
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                dec.replay()
                e.record()
                events.append((s, e))
            else:
                dec.replay()
            run_steps.done += 1
        return events

    run_steps.done = 0
    run_steps(args.warmup, False)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    events = run_steps(args.steps, True)
    barrier()
    total_ms = sum(s.elapsed_time(e) for s, e in events)

    # the same steps without the L2 flush (weights stay L2-resident between positions)
    barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dec.position.fill_(prefix)
    s.record()
    for i in range(min(args.steps, 64)):
        dec.replay()
    e.record()
    torch.cuda.synchronize()
    warm_ms = s.elapsed_time(e) / min(args.steps, 64)

    # end to end: host token ids in, greedy token out, every step
    # (the decoder's host-transfer graph: pinned ids -> device at its head, chosen tokens -> pinned
    # memory at its tail, one launch and one stream synchronisation per position)
    dec.position.fill_(prefix)                          # the capture's warm-up steps run at the current position
    dec.capture_host_io()
    dec.host_tokens.copy_(tokens[:, prefix].cpu())
    dec.host_boundaries.zero_()
    torch.cuda.synchronize()
    e2e_steps = min(args.steps, 64)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        chosen = dec.step_host()
        dec.host_tokens.copy_(chosen)                   # greedy feedback through the host
    e2e_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop() if sampler else None
    assert _abi.read_status() == 0, "a kernel reported a device-side error"

    total_ms, e2e_ms, warm_ms = max_over_ranks([total_ms, e2e_s * 1e3, warm_ms], world, device)

    if rank == 0:
        log(f"timed region done: {total_ms / args.steps:.3f} ms/step")
        table = kernel_table(dec)
        rows256 = select_rows256(device)
        log("kernel table done")
        peaks = {}
        try:
            peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        dominant = max(table, key=lambda k: table[k]["us_per_step"])
        dom = table[dominant]
        lib_us = sum(v["us_per_step"] for v in table.values())
        threads = os.cpu_count() or 1
        cpu_steps = 6
        cpu_batch = min(B, CPU_SAMPLE_BATCH)
        if world == 1:
            log(f"cpu baseline: {cpu_steps} positions of {cpu_batch} sequences on {threads} threads")
            cpu_value, cpu_elapsed, cpu_threads = cpu_decode_rate(args.workload, cpu_batch, cpu_steps, 1, threads)
            cpu_sample = (f"{cpu_steps} decode positions of {cpu_batch} of the {B} sequences from a synthetic "
                          "end-of-prefix state, CPU port of the step (C oracle + fp32 torch matmuls)")
        else:                       # the host cores are busy with the other ranks: measured at N=1 only
            cpu_value, cpu_threads, cpu_sample = None, 0, "not run with more than one GPU rank"
        line = {
            "metric": METRIC, "value": job_rate(world, B, args.steps, total_ms), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {**workload_config(args.workload, B, world),
                       "parameters": model.parameter_count(), "state_bytes_per_gpu": dec.state_bytes()},
            "e2e": {"value": job_rate(world, B, e2e_steps, e2e_ms), "unit": UNIT,
                    "h2d_bytes_per_step": 2 * B * 8, "d2h_bytes_per_step": B * 8,
                    "steps": e2e_steps},
            "gpu_launches": kernels_per_step * args.steps,
            "l2_warm": {"ms_per_step": warm_ms, "value": world * B / (warm_ms / 1e3), "unit": UNIT,
                        "note": "same steps back to back without the L2 flush"},
            "clocks": clocks,
            "roofline": {"kernel": dominant, "bound": "hbm", "achieved": dom["gb_per_s"], "peak": peak,
                         "unit": "GB/s", "frac": dom["gb_per_s"] / peak,
                         "peak_source": "measured" if peaks else "fallback",
                         "traffic": (round(dom["bytes_per_launch"] * NCU_SELECT_TRAFFIC_RATIO)
                                     if dominant == "relation_select_kernel" else None),
                         "traffic_source": "DRAM bytes of the 256-row ncu capture of this kernel (21.46 MB per "
                                           "launch for 21.33 MB of algorithmic bytes), scaled by algorithmic bytes",
                         "us_per_launch": dom["us_per_launch"],
                         "share_of_library_time": dom["us_per_step"] / lib_us,
                         "note": "batch-8 decode launches move < 1 MB each and are latency-bound"},
            "kernels": table,
            "roofline_rows256": {**rows256, "peak": peak, "frac": rows256["gb_per_s"] / peak,
                                 "traffic": NCU_SELECT_TRAFFIC_ROWS256,
                                 "note": "the selector at 256 rows of the 12-layer decode shape, the "
                                         "smallest launch whose bytes (21 MB) are bandwidth-relevant"},
            "cpu_baseline": {"value": cpu_value, "unit": UNIT, "cores": cpu_threads, "kind": "port",
                             "sample": cpu_sample},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def run_kernel_case(args) -> None:
    """A handful of eager launches of one kernel on caches of several layers (hundreds of MB,
    so consecutive launches do not hit L2), at the d_model-768 / ctx-2048 / block-64 decode shape."""
    from relation_lm.kernels.relation_reduce import (relation_hidden_cache_update_out, relation_hidden_cached,
                                                     relation_norm_reduce)
    from relation_lm.kernels.relation_select import relation_select_packed
    from relation_lm.kernels.router_cache import router_cache_update

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    B, T, bs, L, TOP, K, H, R, d = args.rows, args.ctx, 64, 128, 2, 8, 3072, 128, 768
    nb, sets = T // bs, 4
    rn = lambda *s: torch.randn(*s, device=dev).bfloat16()  # noqa: E731
    pos = torch.tensor(T - 1, device=dev)
    events = []
    for i in range(sets + 2):
        if args.kernel_case == "select":
            if i == 0:
                S = [(rn(B, T, 64), rn(B, T, 64), rn(B, T, 128), rn(B, nb, 4, 16), rn(B, nb, 4, 16).abs(),
                      rn(B, nb, 4, 16), rn(B, nb, 4, 16).abs()) for _ in range(sets)]
                q, g, bias = rn(B, 256), torch.randn(4, device=dev), torch.randn(4, 16, device=dev)
            ak, pk, pac, am, as_, pm, ps = S[i % sets]
            fn = lambda: relation_select_packed(q[:, :64], ak, q[:, 64:128], am, as_, g, bias, q[:, 128:],  # noqa: E731
                                                pac, pk, pm, ps, g, bias, pos, L, TOP, K, False)
        elif args.kernel_case == "hidden":
            if i == 0:
                S = [(rn(B, T, 2 * H), rn(B, T, R)) for _ in range(2)]
                wm = rn(H, R) * 0.02
                ai = torch.randint(0, T, (B,), device=dev, dtype=torch.int32)
                pi = torch.randint(0, T, (B, K), device=dev, dtype=torch.int32)
            ex, op = S[i % 2]
            fn = lambda: relation_hidden_cached(ex, op, ai, pi, wm)  # noqa: E731
        elif args.kernel_case == "hidden_update":
            if i == 0:
                S = [(rn(B, T, 2 * H), rn(B, T, R)) for _ in range(2)]
                wm, wa, wp, b1 = rn(H, R) * 0.02, rn(H, R) * 0.02, rn(H, R) * 0.02, rn(H) * 0.01
                ai = torch.randint(0, T, (B,), device=dev, dtype=torch.int32)
                pi = torch.randint(0, T, (B, K), device=dev, dtype=torch.int32)
                hidden_out = torch.empty(B, K, H, device=dev, dtype=torch.bfloat16)
            ex, op = S[i % 2]
            fn = lambda: relation_hidden_cache_update_out(hidden_out, ex, op, ai, pi, wa, wp, wm, b1, pos)  # noqa: E731
        elif args.kernel_case == "projection":
            if i == 0:
                from relation_lm.kernels.packed_projection import packed_projection
                S = [rn(B, d) for _ in range(sets)]
                w_packed = rn(12 * (384 + R), d) * 0.02          # the 12-layer packed projection matrix
            x = S[i % sets]
            fn = lambda: packed_projection(x, w_packed)  # noqa: E731
        elif args.kernel_case == "norm":
            if i == 0:
                S = [rn(B, K, d) for _ in range(sets)]
                sc, gm, bt = torch.randn(B, K, device=dev), torch.ones(d, device=dev), torch.zeros(d, device=dev)
            raw = S[i % sets]
            fn = lambda: relation_norm_reduce(raw, sc, gm, bt, pos, 1e-5)  # noqa: E731
        elif args.kernel_case == "norm_project":
            if i == 0:
                from relation_lm.kernels.relation_reduce import relation_norm_reduce_residual_norm_project
                S = [rn(B, K, d) for _ in range(sets)]
                sc, gm, bt = torch.randn(B, K, device=dev), torch.ones(d, device=dev), torch.zeros(d, device=dev)
                residual, mix = torch.randn(B, d, device=dev), torch.tensor(0.3, device=dev)
                normalized, wq = rn(B, d), rn(256, d) * 0.04
                projected = rn(B, 256)
            raw = S[i % sets]
            fn = lambda: relation_norm_reduce_residual_norm_project(  # noqa: E731
                raw, sc, gm, bt, pos, 1e-5, residual, mix, gm, bt, 1e-5, normalized, wq, projected)
        else:
            if i == 0:
                S = [([rn(B, T, 64) for _ in range(4)], [rn(B, nb, 4, 16) for _ in range(4)]) for _ in range(sets)]
                packed, wc = rn(B, 512), torch.randn(64, 3, device=dev) * 0.1
            caches, stats = S[i % sets]
            fn = lambda: router_cache_update(packed[:, 384:448], packed[:, 448:512], *caches, *stats, wc, wc, pos, bs)  # noqa: E731
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        events.append((s, e))
    torch.cuda.synchronize()
    print(json.dumps({"kernel_case": args.kernel_case, "rows": B,
                      "us": [round(s.elapsed_time(e) * 1e3, 2) for s, e in events]}))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--workload", choices=("cfg2", "cfg5"), default="cfg2")
    parser.add_argument("--batch", type=int, default=None, help="sequences per GPU")
    parser.add_argument("--prefix", type=int, default=None,
                        help="prefix length (default: context - 64); shorter only for profiling runs")
    parser.add_argument("--kernel-case", choices=("select", "hidden", "hidden_update", "projection", "norm", "norm_project", "router"),
                        default=None,
                        help="launch one library kernel a few times at --rows rows of the 12-layer "
                             "decode shape and exit (for profiler captures)")
    parser.add_argument("--rows", type=int, default=256)
    parser.add_argument("--ctx", type=int, default=2048,
                        help="cache length of --kernel-case runs (shorter caches keep profiler captures small)")
    args = parser.parse_args()
    if args.kernel_case:
        run_kernel_case(args)
        return
    if args.batch is None:
        args.batch = 8 if args.workload == "cfg2" else 256 // max(1, args.gpus)
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
