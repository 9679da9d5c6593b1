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
REFERENCE_INSTALL = ROOT / "baseline" / "_ref"        # `pip install --target` of the reference project, if present
# Both this repository's package and the reference's are called `relation_lm` (same module paths,
# same operator names): a process imports one of them.  The sub-process modes that run the
# reference's own code put its install first and leave this repository's package off the path.
_REFERENCE_PROCESS = any(a in ("--op-microbench=reference", "--dense-cpu") for a in sys.argv[1:])
for _p in ((REFERENCE_INSTALL,) if _REFERENCE_PROCESS else (ROOT, ROOT / "relation-lm_b200")):
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
# dram__bytes_read + write of one relation_layer_tail_kernel launch at 8 sequences x K = 8, d 512, hidden 2048
# (ncu capture of `--kernel-case tail --rows 8`), over the algorithmic bytes of the same launch
NCU_TAIL_TRAFFIC_RATIO = 3_298_816 / 3_251_776
# the CPU port keeps fp32 caches on the host (58 MB per sequence at ctx 512 / d 512, 750 MB at ctx 2048 / d 768)
CPU_MAX_BATCH = {"cfg2": 64, "cfg5": 8}


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
        late = not self.samples
        deadline = time.time() + 0.2                    # a region shorter than the sampling period: take the next sample
        while not self.samples and time.time() < deadline:
            time.sleep(0.005)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[3:7]) if v == "Active"})
        record = {"sm_mhz": statistics.median(sm) if sm else None,
                  "sm_max_mhz": float(self.samples[0][1]) if self.samples else None,
                  "samples": len(self.samples), "reasons": reasons}
        if late and self.samples:
            record["note"] = "the timed region was shorter than the 20 ms sampling period: sampled right after it"
        return record


# ---------------------------------------------------------------------------- CPU arm


def cpu_decode_rate(workload: str, batch: int, steps: int, warmup: int, threads: int, runs: int = 1):
    """The CPU port of the decode step on the host cores, from a synthetic state at the end
    of the prefix (cache contents do not change the work done).  `warmup` untimed positions, then
    `runs` timed runs of `steps` positions each; returns the median run's (tokens/s, seconds),
    the threads used and every run's rate."""
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
    total = warmup + runs * steps
    tokens = zipf_tokens(batch, total, cfg.vocab_size, seed)
    bounds = torch.randint(0, cfg.boundary_vocab_size, (batch, total), generator=g)

    def advance(i):
        if dec.position >= cfg.max_context:
            dec.position = prefix
        dec.step(tokens[:, i], bounds[:, i])

    for i in range(warmup):
        advance(i)
    elapsed = []
    for r in range(runs):
        start = time.perf_counter()
        for i in range(warmup + r * steps, warmup + (r + 1) * steps):
            advance(i)
        elapsed.append(time.perf_counter() - start)
    median = statistics.median(elapsed)
    return batch * steps / median, median, threads, [batch * steps / e for e in elapsed]


def run_reference(args) -> None:
    """The reference arm: the CPU implementation of the same decode step on the host cores, all
    threads, decoding the same number of sequences as the GPU arm's whole job (up to
    CPU_MAX_BATCH: the CPU port keeps fp32 caches on the host)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    world = max(1, args.gpus)
    cpu_batch = min(args.batch * world, CPU_MAX_BATCH[args.workload])
    value, elapsed, threads, _ = cpu_decode_rate(args.workload, cpu_batch, steps, args.warmup, 0)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": elapsed / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {**workload_config(args.workload, args.batch, world), "sequences_decoded": cpu_batch},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{steps} decode positions of {cpu_batch} of the job's {args.batch * world} sequences "
                                   "from a synthetic end-of-prefix state, CPU port of the step (C oracle + fp32 torch matmuls)"},
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

    layer_tail = getattr(dec, "layer_tail", False)

    def tail(l):
        from relation_lm.kernels.relation_reduce import relation_layer_tail
        relation_layer_tail(dec.expanded_cache[l], dec.operand_cache[l], anchor, partner, scores,
                            w["product_weight"][l], w["w2"][l], w["b2"][l], w["relation_norm_w"][l],
                            w["relation_norm_b"][l], pos, cfg.norm_eps, residual, w["mix"][l], w["input_norm_w"][l],
                            w["input_norm_b"][l], cfg.norm_eps, normalized, w["w_query"][l], projected)

    def append(_):
        sparse_cache_append(packed, dec.anchor_keys, dec.partner_keys, dec.operand_cache,
                            dec.partner_anchor_cache, *dec.router_caches, *dec.router_stats,
                            w["anchor_conv_weight"], w["partner_conv_weight"], pos, cfg.block_size)

    fused_front = getattr(dec, "fused_front", False)
    norm_rows = [torch.empty(B, d, device=dev, dtype=dec.dtype) for _ in range(2)]

    def front(_):
        from relation_lm.kernels.packed_projection import decode_front
        decode_front(tokens_in, tokens_in % cfg.boundary_vocab_size, w["token_embedding"], w["boundary_embedding"],
                     w["position_embedding"], pos, dec.input_scale, w["memory_norm_w"], w["memory_norm_b"],
                     w["input_norm_w"][0], w["input_norm_b"][0], cfg.norm_eps, dec.front_weight, w["w_packed"].shape[0],
                     norm_rows[0], norm_rows[1], projected)

    def head(_):
        from relation_lm.kernels.packed_projection import skinny_projection
        skinny_projection(normalized, dec.head_weight, dec.head_bias)

    tokens_in = torch.randint(0, cfg.vocab_size, (B,), device=dev)
    cand = cfg.local_window + cfg.top_blocks * cfg.block_size
    nb = cfg.max_context // cfg.block_size
    # bf16 decode launches of at most one row per SM keep both key caches resident when they fit
    resident = (dec.dtype == torch.bfloat16 and B <= 148 and cfg.top_blocks > 0
                and 2 * cfg.max_context * 128 + 4 * nb * 128 + 8192 <= 223 * 1024)
    key_rows = cfg.max_context if resident else cand
    n_head = dec.head_weight.size(0) if getattr(dec, "skinny", False) else 0
    bytes_per_launch = {
        "skinny_front_kernel": e * ((L * (384 + R) + 256) * d + 2 * B * d + B * (L * (384 + R) + 256)) + 8 * B * d,
        "skinny_projection_kernel(head)": e * (n_head * d + B * d + B * n_head),
        "relation_select_kernel": B * (e * (4 * nb * 64 + 2 * key_rows * 64 + 64 + 64 + 128 + 128) + 2 * (4 + 64) * 4 + 8 + 8 * K),
        "relation_hidden_kernel": B * (e * ((1 + K) * H + (1 + K) * R) + 8 + 4 * K + e * K * H) + e * H * R
                                  + (0 if stacked else e * 2 * H * R + B * e * (R + 2 * H)),
        "expanded_row_update_kernel(all layers)": L * (e * 2 * H * R + B * e * (R + 2 * H)),
        "relation_norm_reduce_kernel": B * (e * K * d + 4 * K + 4 * d + 8 * d) + 4 * 3 * d,
        "packed_projection_kernel(query)": e * (B * d + 256 * d + B * 256),
        "relation_norm_reduce_project_kernel": B * (e * K * d + 4 * K + 4 * d + 8 * d) + 4 * 3 * d
                                               + e * (B * d + 256 * d + B * 256),
        "relation_layer_tail_kernel": e * (H * R + d * H + 256 * d) + B * (e * (1 + K) * (H + R) + 8 + 8 * K + 8 * d + e * d + e * 256)
                                      + 4 * 4 * d + e * d,
        "router_cache_update_kernel(all layers)": L * B * (e * 64 * (2 + 4 + 4 + 2 * cfg.block_size + 4) + 2 * 64 * 4 + 2 * e * (256 + R)),
    }
    table = {}
    # (kernel, launcher, launches per timing graph, launches per decode step): with the query
    # projection inside norm-reduce only layer 0 projects separately and only the last layer's
    # norm-reduce runs without a projection
    for name, fn, per_graph, per_step in (
            ("skinny_front_kernel", front, 1, 1),
            ("skinny_projection_kernel(head)", head, 1, 1),
            ("relation_select_kernel", select, L, L),
            ("relation_layer_tail_kernel", tail, L, L),
            ("relation_hidden_kernel", hidden, L, L),
            ("relation_norm_reduce_kernel", reduce, L, 1 if fused_query else L),
            ("relation_norm_reduce_project_kernel", reduce_project, L, L - 1),
            ("packed_projection_kernel(query)", query, L, 1 if (fused_query or layer_tail) else L),
            ("router_cache_update_kernel(all layers)", append, 1, 1),
            ("expanded_row_update_kernel(all layers)", expand, 1, 1)):
        if name.startswith("expanded_row_update") and not stacked:
            continue
        if name == "skinny_front_kernel" and not fused_front:
            continue
        if name == "skinny_projection_kernel(head)" and not n_head:
            continue
        if name == "packed_projection_kernel(query)" and fused_front:
            continue
        if name == "relation_norm_reduce_project_kernel" and not fused_query:
            continue
        if (name == "relation_layer_tail_kernel") != layer_tail and name in (
                "relation_layer_tail_kernel", "relation_hidden_kernel", "relation_norm_reduce_kernel"):
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


def _time_graph(launchers, device, replays: int = 10) -> float:
    """Average device time, in microseconds, of the launches in `launchers` captured back to back
    in one CUDA graph (three warm-up replays, then `replays` timed ones)."""
    launchers[0]()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for fn in launchers:
                fn()
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) * 1e3 / (replays * len(launchers))


L2_BYTES = 126 * 1024 * 1024


def rows256_table(device) -> dict:
    """The three per-row kernels at the row count where bandwidth starts to matter: 256 rows of the
    12-layer decode shape (d_model 768, hidden 3072, block 64, window 128, 2 remote blocks, K 8,
    bf16).  Each kernel rotates through enough independent input sets that the bytes TOUCHED
    between two uses of a set exceed twice the L2 capacity, so every launch reads from DRAM."""
    from relation_lm.kernels.relation_reduce import relation_hidden_cached_out, relation_norm_reduce
    from relation_lm.kernels.relation_select import relation_select_packed

    B, T, bs, L, TOP, K, d, H, R = 256, 2048, 64, 128, 2, 8, 768, 3072, 128
    nb = T // bs
    rn = lambda *shape: torch.randn(*shape, device=device).bfloat16()  # noqa: E731
    pos = torch.tensor(T - 1, device=device)
    table = {}

    def sets_for(bytes_touched: int) -> int:
        return max(3, -(-2 * L2_BYTES // bytes_touched) + 1)

    # selector
    cand = L + TOP * bs
    select_bytes = B * (2 * (4 * nb * 64 + 2 * cand * 64 + 64 + 64 + 128 + 128) + 2 * (4 + 64) * 4 + 8 + 8 * K)
    n = sets_for(select_bytes)
    S = [(rn(B, T, 64), rn(B, T, 64), rn(B, T, 128), rn(B, nb, 4, 16), rn(B, nb, 4, 16).abs(),
          rn(B, nb, 4, 16), rn(B, nb, 4, 16).abs()) for _ in range(n)]
    q, g, bias = rn(B, 256), torch.randn(4, device=device), torch.randn(4, 16, device=device)

    def select(i):
        ak, pk, pac, am, as_, pm, ps = S[i]
        return lambda: relation_select_packed(q[:, :64], ak, q[:, 64:128], am, as_, g, bias, q[:, 128:], pac, pk,
                                              pm, ps, g, bias, pos, L, TOP, K, False)

    us = _time_graph([select(i) for i in range(n)], device)
    table["relation_select_kernel"] = {"us_per_launch": us, "bytes_per_launch": select_bytes, "input_sets": n}
    del S
    # relation hidden, cached form on the tensor cores (a short cache: the gathered rows are random anyway)
    Th = 128
    hidden_bytes = B * (2 * (1 + K) * (H + R) + 8 + 4 * K + 2 * K * H) + 2 * H * R
    n = sets_for(hidden_bytes)
    S = [(rn(B, Th, 2 * H), rn(B, Th, R), torch.empty(B, K, H, device=device, dtype=torch.bfloat16)) for _ in range(n)]
    wm = rn(H, R) * 0.02
    ai = torch.randint(0, Th, (B,), device=device, dtype=torch.int32)
    pi = torch.randint(0, Th, (B, K), device=device, dtype=torch.int32)

    def hidden(i):
        ex, op, out = S[i]
        return lambda: relation_hidden_cached_out(out, ex, op, ai, pi, wm)

    us = _time_graph([hidden(i) for i in range(n)], device)
    table["relation_hidden_tc_kernel"] = {"us_per_launch": us, "bytes_per_launch": hidden_bytes, "input_sets": n}
    del S
    # norm-reduce
    norm_bytes = B * (2 * K * d + 4 * K + 4 * d) + 2 * 4 * d
    n = sets_for(norm_bytes)
    S = [rn(B, K, d) for _ in range(n)]
    sc, gm, bt = torch.randn(B, K, device=device), torch.ones(d, device=device), torch.zeros(d, device=device)
    us = _time_graph([(lambda raw=raw: relation_norm_reduce(raw, sc, gm, bt, pos, 1e-5)) for raw in S], device)
    table["relation_norm_reduce_vec_kernel"] = {"us_per_launch": us, "bytes_per_launch": norm_bytes, "input_sets": n}
    for row in table.values():
        row["rows"] = B
        row["gb_per_s"] = row["bytes_per_launch"] / row["us_per_launch"] / 1e3
    return table


def measure_decode(workload: str, batch: int, args, rank: int, world: int, device, barrier) -> dict:
    """Prefix + timed decode positions of one workload on this rank's sequences; returns the
    pieces of the result line (timings already reduced to the maximum over ranks)."""
    from relation_lm.inference.stateful_decode import StatefulDecoder
    from relation_lm.kernels import _abi

    model, seed = make_model(workload)
    cfg = model.config
    B, T = batch, cfg.max_context
    prefix = T - 64 if args.prefix is None else args.prefix
    dec = StatefulDecoder(model, B, device, torch.bfloat16)
    tokens, bounds = rank_inputs(cfg, seed, B, rank)
    tokens, bounds = tokens.to(device), bounds.to(device)
    log(f"{workload}: state allocated, {dec.state_bytes() / 1e9:.1f} GB")
    launches_before = _abi.launch_count()
    dec.step_greedy(tokens[:, 0], bounds[:, 0])          # what the captured graph replays
    kernels_per_step = _abi.launch_count() - launches_before
    dec.reset()
    dec.capture()
    for t in range(prefix):                              # the prefix, through the captured step
        dec.static_tokens.copy_(tokens[:, t])
        dec.static_boundaries.copy_(bounds[:, t])
        dec.replay()
    torch.cuda.synchronize()
    log(f"{workload}: prefix of {prefix} positions done")
    assert int(dec.position.item()) == prefix
    assert _abi.read_status() == 0, "a kernel reported a device-side error during the prefix"

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    done = [0]

    def run_steps(count: int, timed: bool):
        events = []
        for _ in range(count):
            t = prefix + (done[0] % 64)
            if t == prefix and done[0]:
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
            done[0] += 1
        return events

    run_steps(args.warmup, False)
    barrier()
    events = run_steps(args.steps, True)
    barrier()
    total_ms = sum(s.elapsed_time(e) for s, e in events)

    # the same steps without the L2 flush (weights stay L2-resident between positions)
    barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dec.position.fill_(prefix)
    warm_steps = min(args.steps, 64)
    s.record()
    for _ in range(warm_steps):
        dec.replay()
    e.record()
    torch.cuda.synchronize()
    warm_ms = s.elapsed_time(e) / warm_steps

    # end to end: host token ids in, greedy token out, every step (the decoder's host-transfer
    # graph: pinned ids -> device at its head, chosen tokens -> pinned memory at its tail, one
    # launch and one stream synchronisation per position)
    dec.position.fill_(prefix)                          # the capture's warm-up steps run at the current position
    dec.capture_host_io()
    dec.host_tokens.copy_(tokens[:, prefix].cpu())
    dec.host_boundaries.zero_()
    torch.cuda.synchronize()
    e2e_steps = min(args.steps, 64)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        chosen = dec.step_host()
        dec.host_tokens.copy_(chosen)                   # greedy feedback through the host
    e2e_warm_s = time.perf_counter() - t0
    # the same loop with the L2 flushed before every step, as in the device-timed region: the flush and
    # its synchronisation lie outside the host clock, the step (graph launch, both copies, sync) inside
    dec.position.fill_(prefix)
    dec.host_tokens.copy_(tokens[:, prefix].cpu())
    e2e_s = 0.0
    barrier()
    for _ in range(e2e_steps):
        flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        chosen = dec.step_host()
        e2e_s += time.perf_counter() - t0
        dec.host_tokens.copy_(chosen)
    barrier()
    # decoding past the context: the state slides by one router block whenever the position reaches
    # max_context.  One slide timed alone with a cold L2, and 2 x block_size positions back to back with
    # the two slides they need inside the timed region (compare with l2_warm).
    bs = cfg.block_size
    slide_us = []
    for _ in range(3):
        dec.position.fill_(T)
        flush.zero_()
        flush.zero_()                                   # long enough for the host to have the slide's launch queued
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        dec.slide(1)
        e.record()
        torch.cuda.synchronize()
        slide_us.append(s.elapsed_time(e) * 1e3)
    dec.position.fill_(T)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(2):
        dec.slide(1)
        for _ in range(bs):
            dec.replay()
    e.record()
    torch.cuda.synchronize()
    sliding_ms = s.elapsed_time(e) / (2 * bs)
    assert int(dec.position.item()) == T
    dec.position.fill_(prefix)
    assert _abi.read_status() == 0, "a kernel reported a device-side error"
    total_ms, e2e_ms, e2e_warm_ms, warm_ms = max_over_ranks([total_ms, e2e_s * 1e3, e2e_warm_s * 1e3, warm_ms], world, device)
    moved = dec.state_bytes() * (T - bs) // T
    result = {
        "value": job_rate(world, B, args.steps, total_ms), "ms_per_step": total_ms / args.steps,
        "e2e": {"value": job_rate(world, B, e2e_steps, e2e_ms), "unit": UNIT,
                "h2d_bytes_per_step": 2 * B * 8, "d2h_bytes_per_step": B * 8, "steps": e2e_steps,
                "l2": "flushed before every step (outside the host clock)",
                "l2_warm_value": job_rate(world, B, e2e_steps, e2e_warm_ms),
                "note": "host-timed: pinned ids -> device (one copy node), the step's graph, chosen tokens written into pinned "
                        "host memory by the head kernel, stream sync; "
                        "l2_warm_value is the same loop back to back"},
        "l2_warm": {"ms_per_step": warm_ms, "value": world * B / (warm_ms / 1e3), "unit": UNIT,
                    "note": "same steps back to back without the L2 flush"},
        "sliding": {"blocks_per_slide": 1, "positions_per_slide": bs, "slide_us": sorted(slide_us)[1],
                    "moved_bytes": moved, "gb_per_s": 2 * moved / (sorted(slide_us)[1] * 1e-6) / 1e9,
                    "bound": "hbm", "algorithmic_bytes": 2 * moved,
                    "ms_per_step_with_slides": sliding_ms, "value_with_slides": B / (sliding_ms / 1e3), "unit": UNIT,
                    "note": "past max_context the state slides by one router block every block_size positions "
                            "(state_slide_kernel: every surviving byte read and written once, cold L2 for slide_us); "
                            "value_with_slides is this rank's rate back to back with the slides in the timed region, "
                            "to set beside l2_warm"},
        "gpu_launches": kernels_per_step * args.steps, "launches_per_step": kernels_per_step,
        "parameters": model.parameter_count(), "state_bytes_per_gpu": dec.state_bytes(),
    }
    if rank == 0:
        log(f"{workload}: timed region done, {total_ms / args.steps:.3f} ms/step")
        result["kernels"] = kernel_table(dec)
    del dec, flush
    torch.cuda.empty_cache()
    return result


def roofline_of(table: dict, peak: float, peaks_found: bool) -> dict:
    """The roofline record of the library kernel with the largest share of a decode step."""
    dominant = max(table, key=lambda k: table[k]["us_per_step"])
    dom = table[dominant]
    lib_us = sum(v["us_per_step"] for v in table.values())
    return {"kernel": dominant, "bound": "hbm", "achieved": dom["gb_per_s"], "peak": peak,
            "unit": "GB/s", "frac": dom["gb_per_s"] / peak,
            "peak_source": "measured" if peaks_found else "fallback",
            "traffic": (round(dom["bytes_per_launch"] * NCU_SELECT_TRAFFIC_RATIO) if dominant == "relation_select_kernel"
                        else round(dom["bytes_per_launch"] * NCU_TAIL_TRAFFIC_RATIO) if dominant == "relation_layer_tail_kernel"
                        else None),
            "traffic_source": ("DRAM bytes of the ncu capture of this kernel at 8 sequences (3.30 MB per launch for 3.25 MB "
                               "of algorithmic bytes), scaled by algorithmic bytes" if dominant == "relation_layer_tail_kernel"
                               else "DRAM bytes of the 256-row ncu capture of this kernel (21.46 MB per launch for 21.33 MB "
                                    "of algorithmic bytes), scaled by algorithmic bytes"),
            "us_per_launch": dom["us_per_launch"], "bytes_per_launch": dom["bytes_per_launch"],
            "share_of_library_time": dom["us_per_step"] / lib_us}


def run_subprocess_json(mode: str, timeout: int):
    """Runs `bench.py <mode>` in a child process and parses its one JSON line; a dict with
    "unavailable" on any failure (the child imports the reference's package, which cannot share a
    process with this repository's)."""
    try:
        done = subprocess.run([sys.executable, str(ROOT / "bench.py"), mode], capture_output=True, text=True,
                              timeout=timeout)
        lines = [ln for ln in done.stdout.splitlines() if ln.startswith("{")]
        if done.returncode != 0 or not lines:
            return {"unavailable": (done.stderr.strip().splitlines() or ["no output"])[-1][:200]}
        return json.loads(lines[-1])
    except (subprocess.TimeoutExpired, OSError, ValueError) as exc:
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}


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

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    B = args.batch
    sampler = ClockSampler(local) if rank == 0 else None
    main = measure_decode(args.workload, B, args, rank, world, device, barrier)
    clocks = sampler.stop() if sampler else None
    # the strong-scaling companion: 256 sequences of the 12-layer configuration split over the ranks
    sharded = None
    if args.workload == "cfg2" and not args.no_cfg5 and 256 % world == 0:
        sharded = measure_decode("cfg5", 256 // world, args, rank, world, device, barrier)

    if rank == 0:
        peaks = {}
        try:
            peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        rows256 = rows256_table(device)
        for row in rows256.values():
            row["frac"] = row["gb_per_s"] / peak
        rows256["relation_select_kernel"]["traffic"] = NCU_SELECT_TRAFFIC_ROWS256
        log("kernel tables done")
        threads = os.cpu_count() or 1
        cpu_batch = min(B, CPU_MAX_BATCH[args.workload])
        extras = {}
        if world == 1:
            log(f"cpu baseline: 5 runs of 8 positions of {cpu_batch} sequences on {threads} threads, then on 1")
            cpu_value, _, cpu_threads, cpu_runs = cpu_decode_rate(args.workload, cpu_batch, 8, 2, threads, runs=5)
            one_value, _, _, _ = cpu_decode_rate(args.workload, cpu_batch, 2, 1, 1, runs=3)
            cpu_sample = (f"median of 5 runs of 8 decode positions (2 warm-up positions) of {cpu_batch} of the {B} "
                          "sequences from a synthetic end-of-prefix state, CPU port of the step (C oracle + fp32 torch matmuls)")
            cpu_extra = {"runs": cpu_runs, "one_thread": {"value": one_value, "unit": UNIT, "cores": 1,
                                                          "sample": "median of 3 runs of 2 positions"}}
            if args.no_extras:
                cpu_extra["dense_reference"] = {"unavailable": "skipped (--no-extras)"}
            elif REFERENCE_INSTALL.exists():
                cpu_extra["dense_reference"] = run_subprocess_json("--dense-cpu", 300)
                extras["reference_triton"] = run_subprocess_json("--op-microbench=reference", 420)
                extras["ours_same_protocol"] = run_subprocess_json("--op-microbench=ours", 240)
            else:
                cpu_extra["dense_reference"] = {"unavailable": "the reference install (baseline/_ref) is not present"}
        else:                       # the host cores are busy with the other ranks: measured at N=1 only
            cpu_value, cpu_threads, cpu_sample, cpu_extra = None, 0, "not run with more than one GPU rank", {}
        roofline = roofline_of(main["kernels"], peak, bool(peaks))
        roofline["note"] = "batch-8 decode launches move < 1 MB each and are latency-bound"
        line = {
            "metric": METRIC, "value": main["value"], "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {**workload_config(args.workload, B, world),
                       "parameters": main["parameters"], "state_bytes_per_gpu": main["state_bytes_per_gpu"]},
            "e2e": main["e2e"], "gpu_launches": main["gpu_launches"], "launches_per_step": main["launches_per_step"],
            "l2_warm": main["l2_warm"], "sliding": {**main["sliding"], "peak": peak, "frac": main["sliding"]["gb_per_s"] / peak},
            "clocks": clocks, "roofline": roofline,
            "kernels": main["kernels"],
            "roofline_rows256": {**rows256["relation_select_kernel"], "kernel": "relation_select_kernel", "peak": peak,
                                 "note": "the selector at 256 rows of the 12-layer decode shape, the smallest launch "
                                         "whose bytes (21 MB) are bandwidth-relevant; input sets rotated so that "
                                         "every launch misses L2"},
            "rows256": rows256,
            "cpu_baseline": {"value": cpu_value, "unit": UNIT, "cores": cpu_threads, "kind": "port",
                             "sample": cpu_sample, **cpu_extra},
            **extras,
        }
        if sharded is not None:
            line["cfg5"] = {
                "workload": workload_config("cfg5", 256 // world, world)["workload"], "scaling": "strong",
                "global_batch": 256, "batch_per_gpu": 256 // world, "value": sharded["value"], "unit": UNIT,
                "ms_per_step": sharded["ms_per_step"], "e2e": sharded["e2e"], "l2_warm": sharded["l2_warm"],
                "launches_per_step": sharded["launches_per_step"],
                "state_bytes_per_gpu": sharded["state_bytes_per_gpu"],
                "roofline": roofline_of(sharded["kernels"], peak, bool(peaks)), "kernels": sharded["kernels"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------- whole-sequence (prefill) workload


def run_prefill(args) -> None:
    """`--workload cfg3`: relation_select + relation_reduce over whole sequences — batch 8, context
    4096, d_model 512, block 64, window 128, 4 remote blocks, K 8, bf16, hidden states N(0, 1) with
    5 % of the positions scaled by 4 (seeded).  One step = one pass of the routed layer over all
    `batch x 4096` query rows (LayerNorm, query projection, per-row selection, relation hidden,
    second MLP layer, norm-reduce, residual); the sequences' caches and block statistics are
    built once before the timed region (their build time is reported).  Sequences are sharded
    over the ranks."""
    from relation_lm.inference.prefill import RoutedPrefillLayer
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM
    from relation_lm.kernels import _abi
    from relation_lm.kernels.packed_projection import packed_projection
    from relation_lm.kernels.relation_reduce import relation_hidden_cached_rows_out, relation_norm_reduce_rows
    from relation_lm.kernels.relation_select import relation_select_packed_prefill, relation_select_packed_rows

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    T, d = 4096, 512
    cfg = RoutedRelationConfig(vocab_size=64, boundary_vocab_size=8, d_model=d, layers=1, max_context=T,
                               block_size=64, local_window=128, top_blocks=4, k_max=8)
    layer = RoutedPrefillLayer(RoutedRelationLM(cfg, seed=1003), 0, device, torch.bfloat16)
    B = max(1, 8 // world)
    g = torch.Generator().manual_seed(1003 + rank)
    x = torch.randn(B, T, d, generator=g)
    strong = torch.rand(B, T, generator=g) < 0.05
    x = torch.where(strong[..., None], x * 4.0, x).to(device)
    N, K, H = B * T, cfg.k_max, cfg.hidden_dim

    def timed(fn, repeats=1):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(repeats):
            out = fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / repeats, out

    layer.build_state(x)                                     # warm-up of every kernel of the build
    build_ms, state = timed(lambda: layer.build_state(x))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    for _ in range(max(3, args.warmup)):
        layer.forward(x, state)
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    events = []
    for _ in range(args.steps):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        layer.forward(x, state)
        e.record()
        events.append((s, e))
    barrier()
    total_ms = sum(s.elapsed_time(e) for s, e in events)
    clocks = sampler.stop() if sampler else None
    # end to end: the hidden states come from pinned host memory and the layer's output goes back
    host_in = x.cpu().pin_memory()
    host_out = torch.empty_like(host_in).pin_memory()
    dev_in = torch.empty_like(x)
    e2e_steps = min(args.steps, 8)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        dev_in.copy_(host_in, non_blocking=True)
        host_out.copy_(layer.forward(dev_in, state), non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    assert _abi.read_status() == 0, "a kernel reported a device-side error"
    total_ms, e2e_ms, build_ms = max_over_ranks([total_ms, e2e_ms, build_ms], world, device)
    if rank == 0:
        keep: dict = {}
        layer.forward(x, state, keep)
        w = layer.w
        q, rb, rp = keep["query"], keep["row_batch"], keep["row_position"]
        hidden_rel = torch.empty(N, K, H, device=device, dtype=torch.bfloat16)
        select_args = (q[:, 0:64], state["anchor_keys"], q[:, 64:128], state["anchor_mean"], state["anchor_std"],
                       w["anchor_gamma"], w["anchor_bias"], q[:, 128:256], state["partner_anchor_cache"],
                       state["partner_keys"], state["partner_mean"], state["partner_std"], w["partner_gamma"],
                       w["partner_bias"])
        parts = {
            "relation_select_tile_kernel": lambda: relation_select_packed_prefill(
                *select_args, T, cfg.local_window, cfg.top_blocks, K, cfg.strict_valid),
            "relation_select_kernel(rows)": lambda: relation_select_packed_rows(
                *select_args, rb, rp, cfg.local_window, cfg.top_blocks, K, cfg.strict_valid),
            "relation_hidden_tc_kernel(rows)": lambda: relation_hidden_cached_rows_out(
                hidden_rel, state["expanded_cache"], state["operand_cache"], keep["anchor"], keep["partner"],
                w["product_weight"], rb),
            "packed_projection_kernel(second layer)": lambda: packed_projection(hidden_rel.view(N * K, H), w["w2"], w["b2"]),
            "relation_norm_reduce_kernel(rows)": lambda: relation_norm_reduce_rows(
                keep["raw"], keep["partner_score"], w["relation_norm_w"], w["relation_norm_b"], rp, cfg.norm_eps),
        }
        kernels = {}
        for name, fn in parts.items():
            fn()
            ms, _ = timed(fn, repeats=5)
            kernels[name] = {"us_per_launch": ms * 1e3}
        peaks = {}
        try:
            peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        nb, cand = T // cfg.block_size, cfg.local_window + cfg.top_blocks * cfg.block_size
        logical = N * (2 * (4 * nb * 64 + 2 * cand * 64 + 384) + 560 + 8 + 8 * K)
        compulsory = 2 * (B * T * (64 + 64 + 128) + 4 * B * nb * 64 + N * 256) + N * (8 + 8 * K)
        flops = N * 2 * (2 * cand * 64 + 2 * 2 * nb * 64)
        fma_peak = 148 * 128 * 2 * (float(peaks.get("sm_max_mhz", 1965.0)) * 1e6) / 1e12
        for name in ("relation_select_tile_kernel", "relation_select_kernel(rows)"):
            us = kernels[name]["us_per_launch"]
            kernels[name].update(
                compulsory_bytes=compulsory, logical_bytes=logical, fp32_flops=flops,
                compulsory_gb_per_s=compulsory / us / 1e3, logical_gb_per_s=logical / us / 1e3,
                tflops=flops / us / 1e6, frac_of_fp32_fma_peak=flops / us / 1e6 / fma_peak)
        kernels["relation_select_kernel(rows)"]["note"] = "the per-row form, not on the pass's path: timed for comparison"
        sel_us = kernels["relation_select_tile_kernel"]["us_per_launch"]
        kernels["relation_hidden_tc_kernel(rows)"]["tflops"] = 2 * N * K * cfg.relation_dim * H / kernels["relation_hidden_tc_kernel(rows)"]["us_per_launch"] / 1e6
        kernels["packed_projection_kernel(second layer)"]["tflops"] = 2 * N * K * H * d / kernels["packed_projection_kernel(second layer)"]["us_per_launch"] / 1e6
        dominant = max((k for k in kernels if k != "relation_select_kernel(rows)"), key=lambda k: kernels[k]["us_per_launch"])
        line = {
            "metric": "relation prefill tokens/s at ctx4096 K=8", "value": world * N * args.steps / (total_ms / 1e3),
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg3 relation_select + relation_reduce prefill: batch 8, ctx 4096, d_model 512, "
                                   "block 64, window 128, 4 remote blocks, 1 anchor, K=8, 5% strong-anchor positions",
                       "batch_per_gpu": B, "global_batch": B * world, "rows_per_step": world * N,
                       "l2": "flushed between steps", "state_build_ms": build_ms},
            "e2e": {"value": world * N * e2e_steps / (e2e_ms / 1e3), "unit": UNIT,
                    "h2d_bytes_per_step": N * d * 4, "d2h_bytes_per_step": N * d * 4, "steps": e2e_steps},
            "gpu_launches": 6 * args.steps, "clocks": clocks, "kernels": kernels,
            "roofline": {"kernel": "relation_select_tile_kernel", "bound": "hbm", "achieved": compulsory / sel_us / 1e3,
                         "peak": peak, "unit": "GB/s", "frac": compulsory / sel_us / 1e3 / peak,
                         "peak_source": "measured" if peaks else "fallback", "traffic": None,
                         "note": "compulsory bytes (every input and output tensor once); the selector's work is fp32 dot "
                                 "products on cache rows that stay in L2: logical bytes and the fp32 FMA fraction are in `kernels`",
                         "dominant_kernel_of_the_pass": dominant},
        }
        if world == 1:
            line["cpu_baseline"] = cpu_prefill_rate(layer, state, keep)
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def run_multi_anchor(args) -> None:
    """`--workload cfg4`: a `RelationBlockStack`-shaped routed multi-anchor stack — depth 4, batch 16,
    context 2048, d_model 512, 4 distinct anchors per query each choosing 4 partners, all anchors
    barred from all partner sets, block 32, 3 remote blocks, bf16, N(0, 1) inputs, random-init
    weights.  One step = the whole stack over all `batch x 2048` query rows: per layer the memory-side
    projection and state build, then the routed pass.  Sequences are sharded over the ranks."""
    from relation_lm.inference.multi_anchor import MultiAnchorConfig, MultiAnchorPrefill, MultiAnchorRoutedStack
    from relation_lm.kernels import _abi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    cfg = MultiAnchorConfig()
    stack = MultiAnchorRoutedStack(cfg, seed=1004)
    runner = MultiAnchorPrefill(stack, device, torch.bfloat16)
    B, T, d = max(1, 16 // world), cfg.max_context, cfg.d_model
    g = torch.Generator().manual_seed(1004 + rank)
    hidden = torch.randn(B, T, d, generator=g).to(device)
    memory = torch.randn(B, T, d, generator=g).bfloat16().to(device)
    N = B * T
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    launches_before = _abi.launch_count()
    runner.forward(hidden, memory)
    launches = _abi.launch_count() - launches_before
    for _ in range(max(3, args.warmup) - 1):
        runner.forward(hidden, memory)
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    events = []
    for _ in range(args.steps):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        runner.forward(hidden, memory)
        e.record()
        events.append((s, e))
    barrier()
    total_ms = sum(s.elapsed_time(e) for s, e in events)
    clocks = sampler.stop() if sampler else None
    host_in = hidden.cpu().pin_memory()
    host_out = torch.empty_like(host_in).pin_memory()
    dev_in = torch.empty_like(hidden)
    e2e_steps = min(args.steps, 8)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        dev_in.copy_(host_in, non_blocking=True)
        host_out.copy_(runner.forward(dev_in, memory), non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    assert _abi.read_status() == 0, "a kernel reported a device-side error"
    total_ms, e2e_ms = max_over_ranks([total_ms, e2e_ms], world, device)
    if rank == 0:
        # per-stage times of the first layer
        stages = {}

        def stage(name, fn):
            fn()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = fn()
            e.record()
            torch.cuda.synchronize()
            stages[name] = {"ms": s.elapsed_time(e)}
            return out

        state = stage("state build (projection, per-slot caches, router prefill, expanded cache)",
                      lambda: runner.build_state(0, memory))
        work = hidden.clone()
        keep: dict = {}
        stage("routed pass (norm, query projection, multi-anchor selection, hidden, second layer, norm-reduce, mix)",
              lambda: runner.forward_layer(0, work, state, keep))
        from relation_lm.kernels.multi_select import relation_select_multi_prefill, relation_select_multi_rows
        w = runner.layers[0]
        S, K = cfg.anchors_per_block, cfg.partners_per_anchor
        q = keep["query"]
        select_args = (q[:, :S * 64].unflatten(1, (S, 64)), state["anchor_keys"], q[:, S * 64:S * 128].unflatten(1, (S, 64)),
                       state["anchor_mean"], state["anchor_std"], w["anchor_gamma"], w["anchor_bias"],
                       q[:, S * 128:].unflatten(1, (S, 128)), state["partner_anchor_cache"], state["partner_keys"],
                       state["partner_mean"], state["partner_std"], w["partner_gamma"], w["partner_bias"])
        stage("relation_select_multi_tile_kernel", lambda: relation_select_multi_prefill(
            *select_args, T, cfg.local_window, cfg.top_blocks, K, cfg.strict_valid))
        stage("relation_select_multi_kernel", lambda: relation_select_multi_rows(
            *select_args, keep["row_batch"], keep["row_position"], cfg.local_window, cfg.top_blocks, K, cfg.strict_valid))
        stages["relation_select_multi_kernel"]["note"] = "the per-row form, not on the pass's path: timed for comparison"
        peaks = {}
        try:
            peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        nb, cand = T // cfg.block_size, cfg.local_window + cfg.top_blocks * cfg.block_size
        logical = N * S * (2 * (4 * nb * 64 + 2 * cand * 64 + 384) + 560 + 8 + 8 * K)
        compulsory = 2 * S * (B * T * (64 + 64 + 128) + 4 * B * nb * 64) + 2 * N * S * 256 + N * S * (9 + 8 * K)
        for name in ("relation_select_multi_tile_kernel", "relation_select_multi_kernel"):
            ms = stages[name]["ms"]
            stages[name].update(compulsory_bytes=compulsory, logical_bytes=logical,
                                compulsory_gb_per_s=compulsory / ms / 1e6, logical_gb_per_s=logical / ms / 1e6)
        sel_ms = stages["relation_select_multi_tile_kernel"]["ms"]
        line = {
            "metric": "multi-anchor relation stack tokens/s at ctx2048, 4 anchors x 4 partners, depth 4",
            "value": world * N * args.steps / (total_ms / 1e3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg4 routed MultiAnchorRelationBlock stack: depth 4, batch 16, ctx 2048, d_model 512, "
                                   "4 anchors x 4 partners, block 32, window 64, 3 remote blocks",
                       "batch_per_gpu": B, "global_batch": B * world, "rows_per_step": world * N,
                       "l2": "flushed between steps"},
            "e2e": {"value": world * N * e2e_steps / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": N * d * 4,
                    "d2h_bytes_per_step": N * d * 4, "steps": e2e_steps},
            "gpu_launches": launches * args.steps, "launches_per_step": launches, "clocks": clocks, "stages_layer0": stages,
            "roofline": {"kernel": "relation_select_multi_tile_kernel", "bound": "hbm", "achieved": compulsory / sel_ms / 1e6,
                         "peak": peak, "unit": "GB/s", "frac": compulsory / sel_ms / 1e6 / peak,
                         "peak_source": "measured" if peaks else "fallback", "traffic": None,
                         "note": "compulsory bytes; the selector's caches stay in L2 and it is bound by instruction issue (logical bytes in stages_layer0)"},
        }
        if world == 1:
            line["cpu_baseline"] = cpu_multi_anchor_rate(stack, runner, state, keep)
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def cpu_multi_anchor_rate(stack, runner, state, keep, sample: int = 256) -> dict:
    """The CPU port's routed multi-anchor selection on a bounded sample of one layer's query rows
    (the selection dominates the CPU time), all host threads."""
    import oracle
    from oracle.multi_anchor_port import OracleMultiAnchor

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    oracle.set_threads(threads)
    port = OracleMultiAnchor(stack, torch.bfloat16)
    g = torch.Generator().manual_seed(6)
    n_rows = keep["query"].size(0)
    rows = torch.randint(0, n_rows, (sample,), generator=g)
    cpu_state = {k: v.float().cpu() for k, v in state.items() if k != "packed"}
    q = keep["query"].cpu()[rows]
    start = time.perf_counter()
    port.select(0, q, cpu_state, keep["row_batch"].cpu()[rows], keep["row_position"].cpu()[rows])
    elapsed = time.perf_counter() - start
    depth = stack.config.depth
    return {"value": sample / (elapsed * depth), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{sample} of the {n_rows} query rows of one layer: oracle multi-anchor selection; "
                      f"tokens/s = rows / (time x {depth} layers)"}


def cpu_prefill_rate(layer, state, keep, sample: int = 1024) -> dict:
    """The CPU oracle on a bounded sample of the same query rows (selection, relation hidden, second
    MLP layer, norm-reduce), all host threads; tokens/s = sampled rows / time."""
    import oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    oracle.set_threads(threads)
    cfg = layer.config
    wc = {k: v.float().cpu() for k, v in layer.w.items()}
    g = torch.Generator().manual_seed(5)
    n_rows = keep["query"].size(0)
    rows = torch.randint(0, n_rows, (sample,), generator=g)
    q = keep["query"].cpu()[rows]
    rb, rp = keep["row_batch"].cpu()[rows], keep["row_position"].cpu()[rows]
    caches = {n: state[n].float().cpu() for n in ("anchor_keys", "partner_keys", "partner_anchor_cache", "anchor_mean",
                                                   "anchor_std", "partner_mean", "partner_std", "expanded_cache",
                                                   "operand_cache")}
    start = time.perf_counter()
    anchor, _, partner, score, _ = oracle.relation_select(
        q[:, 0:64], caches["anchor_keys"], q[:, 64:128], caches["anchor_mean"], caches["anchor_std"],
        wc["anchor_gamma"], wc["anchor_bias"], q[:, 128:256], caches["partner_anchor_cache"], caches["partner_keys"],
        caches["partner_mean"], caches["partner_std"], wc["partner_gamma"], wc["partner_bias"], 0,
        cfg.local_window, cfg.top_blocks, cfg.k_max, cfg.strict_valid, row_batch=rb, row_pos=rp)
    hidden, _ = oracle.relation_hidden(caches["expanded_cache"], caches["operand_cache"], anchor,
                                       partner.clamp(0, cfg.max_context - 1), wc["product_weight"], row_batch=rb, row_pos=rp)
    raw = hidden @ wc["w2"].T + wc["b2"]
    oracle.relation_norm_reduce(raw, score, wc["relation_norm_w"], wc["relation_norm_b"], 0, cfg.norm_eps, row_pos=rp)
    elapsed = time.perf_counter() - start
    return {"value": sample / elapsed, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{sample} of the {n_rows} query rows: oracle selection + relation hidden + second layer + norm-reduce"}


# ---------------------------------------------------------------------------- reference-side child modes


def run_op_microbench(which: str) -> None:
    """The four reference-shaped operators at the ctx-512 decode shapes (batch 1 and 8, bf16
    caches), timed with the reference's own microbenchmark protocol (50 warm-up calls, 400 timed
    calls back to back between two CUDA events: benchmarks/benchmark_relation_select.py:96-107 of
    the reference project) and, where the operator can be captured, as 20 launches inside a CUDA
    graph.  Both packages expose the same module paths and signatures, so this one function times
    whichever `relation_lm` the process imports: the reference's Triton operators JIT-compiled on
    this GPU, or this repository's CUDA library."""
    from relation_lm.kernels.relation_reduce import relation_hidden_cached, relation_norm_reduce
    from relation_lm.kernels.relation_select import relation_select_packed
    from relation_lm.kernels.router_cache import router_cache_update

    dev = torch.device("cuda", 0)
    torch.manual_seed(17)
    T, NB, L, TOP, K, d, H, R = 512, 16, 64, 2, 8, 512, 2048, 128
    bs = T // NB
    rn = lambda *shape: torch.randn(*shape, device=dev).bfloat16()  # noqa: E731

    def eager_us(fn, warmup=50, repeats=400):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(repeats):
            fn()
        end.record()
        end.synchronize()
        return start.elapsed_time(end) * 1e3 / repeats

    def graph_us(fn):
        try:
            return _time_graph([fn] * 20, dev, replays=20)
        except Exception as exc:  # noqa: BLE001 - a JIT operator that cannot be captured is reported, not fatal
            torch.cuda.synchronize()
            return f"not captured: {type(exc).__name__}"

    out = {"package": which, "protocol": "50 warm-up + 400 timed eager calls; 20 launches per CUDA graph x 20 replays",
           "shape": "ctx 512, block 32, window 64, 2 remote blocks, K 8, d 512, hidden 2048, bf16"}
    for batch in (1, 8):
        pos = torch.tensor(T - 1, device=dev, dtype=torch.long)
        sel = (rn(batch, 64), rn(batch, T, 64), rn(batch, 64), rn(batch, NB, 4, 16), rn(batch, NB, 4, 16).abs(),
               torch.randn(4, device=dev), torch.randn(4, 16, device=dev), rn(batch, 128), rn(batch, T, 128),
               rn(batch, T, 64), rn(batch, NB, 4, 16), rn(batch, NB, 4, 16).abs(), torch.randn(4, device=dev),
               torch.randn(4, 16, device=dev))
        packed = rn(batch, 512)
        caches = [rn(batch, T, 64) for _ in range(4)]
        stats = [rn(batch, NB, 4, 16) for _ in range(4)]
        conv = torch.randn(64, 3, device=dev) * 0.1
        expanded, operand, wm = rn(batch, T, 2 * H), rn(batch, T, R), rn(H, R) * 0.02
        ai = torch.randint(0, T, (batch,), device=dev, dtype=torch.int32)
        pi = torch.randint(0, T, (batch, K), device=dev, dtype=torch.int32)
        raw, scores = rn(batch, K, d), torch.randn(batch, K, device=dev)
        gm, bt = torch.ones(d, device=dev), torch.zeros(d, device=dev)
        ops = {
            "relation_select_packed": lambda: relation_select_packed(*sel, pos, L, TOP, K, False),
            "router_cache_update": lambda: router_cache_update(packed[:, 384:448], packed[:, 448:512], *caches,
                                                               *stats, conv, conv, pos, bs),
            "relation_hidden_cached": lambda: relation_hidden_cached(expanded, operand, ai, pi, wm),
            "relation_norm_reduce": lambda: relation_norm_reduce(raw, scores, gm, bt, pos, 1e-5),
        }
        for name, fn in ops.items():
            out[f"{name}_b{batch}"] = {"eager_us": eager_us(fn), "graph_us": graph_us(fn)}
    print(json.dumps(out), flush=True)


def run_dense_cpu() -> None:
    """The reference's own eager CPU code at the ctx-512 decode shape (fp32, batch 8): one dense
    `RelationBlock.forward` over the whole sequence (models/stacked_relation.py:65-136) and one
    `DistilledBlockRouter.anchor_scores` (routing/block_router.py:103-110) — its only CPU
    implementation of the selection / reduction semantics.  2 warm-ups, median of 5 runs."""
    from relation_lm.models.stacked_relation import RelationBlock, RelationBlockConfig
    from relation_lm.routing.block_router import BlockRouterConfig, DistilledBlockRouter

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    torch.manual_seed(1002)
    B, T, d, layers = 8, 512, 512, 6
    block = RelationBlock(RelationBlockConfig(d_model=d, hidden_dim=4 * d)).eval()
    router = DistilledBlockRouter(BlockRouterConfig(d_model=d, block_size=32)).eval()
    hidden, memory = torch.randn(B, T, d), torch.randn(B, T, d)

    def median_ms(fn):
        with torch.no_grad():
            for _ in range(2):
                fn()
            times = []
            for _ in range(5):
                t0 = time.perf_counter()
                fn()
                times.append((time.perf_counter() - t0) * 1e3)
        return statistics.median(times)

    block_ms = median_ms(lambda: block(hidden, memory))
    router_ms = median_ms(lambda: router.anchor_scores(hidden, memory))
    print(json.dumps({
        "kind": "reference", "cores": threads, "dtype": "f32",
        "relation_block_forward_ms": block_ms, "router_anchor_scores_ms": router_ms,
        "value": B * T / (layers * block_ms / 1e3), "unit": UNIT,
        "sample": f"dense forward of one RelationBlock over {B} x {T} positions (d {d}), median of 5 after 2 warm-ups; "
                  f"tokens/s = {B} x {T} positions / ({layers} layers x that time)"}), flush=True)


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
        elif args.kernel_case in ("projection_rows", "second_layer_rows"):
            if i == 0:
                from relation_lm.kernels.packed_projection import packed_projection
                # the packed projection of a 4096-position state build (12 layers, d 768), or the second
                # relation-MLP layer of a whole-sequence pass (262 144 pairs, hidden 2048 -> d 512)
                Mp, Kp, Np = (4096, 768, 6144) if args.kernel_case == "projection_rows" else (262144, 2048, 512)
                S = [rn(Mp, Kp) for _ in range(2)]
                w_rows = rn(Np, Kp) * 0.02
            x = S[i % 2]
            fn = lambda: packed_projection(x, w_rows)  # noqa: E731
        elif args.kernel_case == "tail":
            if i == 0:
                from relation_lm.kernels.relation_reduce import relation_layer_tail
                Bt, Tt, dt_, Ht = min(B, 64), 512, 512, 2048     # the 6-layer decode configuration's layer
                S = [(rn(Bt, Tt, 2 * Ht), rn(Bt, Tt, R), rn(Ht, R) * 0.05, rn(dt_, Ht) * 0.03, rn(256, dt_) * 0.05)
                     for _ in range(sets)]
                b2, gm, bt = rn(dt_) * 0.1, torch.ones(dt_, device=dev), torch.zeros(dt_, device=dev)
                ai = torch.randint(0, Tt, (Bt,), device=dev, dtype=torch.int32)
                pi = torch.randint(0, Tt, (Bt, K), device=dev, dtype=torch.int32)
                sc = torch.randn(Bt, K, device=dev)
                residual, mix = torch.randn(Bt, dt_, device=dev), torch.tensor(0.2, device=dev)
                normalized, query = rn(Bt, dt_), rn(Bt, 256)
                pos = torch.tensor(Tt - 1, device=dev)
            ex, op, wm, w2, wq = S[i % sets]
            fn = lambda: relation_layer_tail(ex, op, ai, pi, sc, wm, w2, b2, gm, bt, pos, 1e-5, residual, mix,  # noqa: E731
                                             gm, bt, 1e-5, normalized, wq, query)
        elif args.kernel_case == "head":
            if i == 0:
                from relation_lm.kernels.packed_projection import skinny_argmax_scratch_bytes, skinny_projection_greedy
                Bh = min(B, 16)
                S = [rn(16640, 512) * 0.05 for _ in range(sets)]          # vocabulary + boundary heads, d 512
                xh, bias = rn(Bh, 512), torch.zeros(16640, device=dev)
                scratch = torch.zeros(skinny_argmax_scratch_bytes(), dtype=torch.uint8, device=dev)
                posh = torch.zeros((), dtype=torch.int64, device=dev)
            wh = S[i % sets]
            fn = lambda: skinny_projection_greedy(xh, wh, bias, 16000, scratch, posh)  # noqa: E731
        elif args.kernel_case == "select_tile":
            if i == 0:
                from relation_lm.kernels.relation_select import relation_select_packed_prefill
                Bs, Ts, nbs = 8, 4096, 64                              # the long-context configuration
                S = [(rn(Bs, Ts, 64), rn(Bs, Ts, 64), rn(Bs, Ts, 128), rn(Bs, nbs, 4, 16), rn(Bs, nbs, 4, 16).abs(),
                      rn(Bs, nbs, 4, 16), rn(Bs, nbs, 4, 16).abs()) for _ in range(2)]
                q, g, bias = rn(Bs * Ts, 256), torch.randn(4, device=dev), torch.randn(4, 16, device=dev)
            ak, pk, pac, am, as_, pm, ps = S[i % 2]
            fn = lambda: relation_select_packed_prefill(q[:, :64], ak, q[:, 64:128], am, as_, g, bias, q[:, 128:],  # noqa: E731
                                                        pac, pk, pm, ps, g, bias, Ts, 128, 4, K, False)
        elif args.kernel_case == "hidden_rows":
            if i == 0:
                from relation_lm.kernels.relation_reduce import relation_hidden_cached_rows_out
                Bs, Ts, Hs = 8, 4096, 2048                             # the long-context configuration (d_model 512)
                Ns = Bs * Ts
                ex, op, wm = rn(Bs, Ts, 2 * Hs) * 0.3, rn(Bs, Ts, R), rn(Hs, R) * 0.05
                rows = torch.arange(Ns, device=dev, dtype=torch.int32) // Ts
                at = torch.arange(Ns, device=dev, dtype=torch.int32) % Ts
                ai = (torch.rand(Ns, device=dev) * (at + 1)).int().clamp(max=Ts - 1)
                pi = (torch.rand(Ns, K, device=dev) * (at[:, None] + 1)).int().clamp(max=Ts - 1)
                hidden_out = torch.empty(Ns, K, Hs, device=dev, dtype=torch.bfloat16)      # 1.07 GB: larger than L2
            fn = lambda: relation_hidden_cached_rows_out(hidden_out, ex, op, ai, pi, wm, rows)  # noqa: E731
        elif args.kernel_case == "slide":
            if i == 0:
                # the state of the 6-layer d-512 decode shape (ctx 512, block 32) for --rows sequences, two sets
                from relation_lm.kernels.router_cache import state_slide
                S = [[rn(6, B, 512, w) for w in (64, 64, 128, 128, 4096, 64, 64, 64, 64)] +
                     [rn(6, B, 16, 4, 16) for _ in range(4)] for _ in range(2)]
            state = S[i % 2]
            fn = lambda: state_slide(state, [32] * 9 + [1] * 4, row_dim=[-2] * 9 + [-3] * 4)  # noqa: E731
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
    parser.add_argument("--workload", choices=("cfg2", "cfg5", "cfg3", "cfg4"), default="cfg2")
    parser.add_argument("--batch", type=int, default=None, help="sequences per GPU")
    parser.add_argument("--prefix", type=int, default=None,
                        help="prefix length (default: context - 64); shorter only for profiling runs")
    parser.add_argument("--kernel-case", choices=("select", "hidden", "hidden_update", "projection", "norm", "norm_project", "router",
                                                 "tail", "head", "select_tile", "hidden_rows", "projection_rows", "second_layer_rows", "slide"),
                        default=None,
                        help="launch one library kernel a few times at --rows rows of the 12-layer "
                             "decode shape and exit (for profiler captures)")
    parser.add_argument("--rows", type=int, default=256)
    parser.add_argument("--ctx", type=int, default=2048,
                        help="cache length of --kernel-case runs (shorter caches keep profiler captures small)")
    parser.add_argument("--no-extras", action="store_true",
                        help="skip the child-process legs (the reference's Triton operators and dense CPU modules): "
                             "for profiler runs, which would otherwise list their launches too")
    parser.add_argument("--no-cfg5", action="store_true",
                        help="skip the 256-sequence 12-layer companion measurement of the default run")
    parser.add_argument("--op-microbench", choices=("ours", "reference"), default=None,
                        help="child mode: time the four reference-shaped operators of one package")
    parser.add_argument("--dense-cpu", action="store_true",
                        help="child mode: time the reference's dense eager CPU modules (needs baseline/_ref)")
    args = parser.parse_args()
    if args.op_microbench:
        run_op_microbench(args.op_microbench)
        return
    if args.dense_cpu:
        run_dense_cpu()
        return
    if args.kernel_case:
        run_kernel_case(args)
        return
    if args.workload == "cfg3":
        run_prefill(args)
        return
    if args.workload == "cfg4":
        run_multi_anchor(args)
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
