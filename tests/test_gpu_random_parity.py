"""Seeded random configurations against the CPU oracle: shapes, policies, positions and dtypes that the
hand-picked cases do not list.  Selectors (decode form, per-row form, whole-sequence tile form): indices
and scores bit-exact.  Relation hidden / norm-reduce: 2e-5 in fp32, 1e-2 of the row's largest magnitude
with 16-bit operands.  Router update: bit-exact on all eight state tensors.  Relation layer tail: 1e-2 of
the row's largest magnitude and bit-identical on a second call."""
from __future__ import annotations

import random

import pytest
import torch

import cases
import oracle
from gpu_util import SELECT_KEYS, assert_status_clear, position_tensor, select_args, to_cuda

pytestmark = pytest.mark.gpu

DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def _bits(x: torch.Tensor) -> torch.Tensor:
    return torch.nan_to_num(x.float().cpu(), neginf=-1.0e38).view(torch.int32)


def _same_selection(got, want) -> bool:
    return (torch.equal(got[0].cpu(), want[0].cpu()) and torch.equal(got[2].cpu(), want[2].cpu())
            and torch.equal(_bits(got[1]), _bits(want[1])) and torch.equal(_bits(got[3]), _bits(want[3])))


def _close(got, want, low) -> bool:
    got, want = got.float().cpu(), want.float()
    if low:
        scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1.0e-6)
        return bool(((got - want).abs() <= 1.0e-2 * scale + 1.0e-6).all())
    return torch.allclose(got, want, atol=2.0e-5, rtol=1.0e-5)


def test_random_selector_configurations():
    from relation_lm.kernels.relation_select import (relation_select_packed, relation_select_packed_prefill,
                                                     relation_select_packed_rows)

    rng = random.Random(20261)
    done = 0
    while done < 500:
        bs, nb = rng.choice([8, 16, 32, 64]), rng.choice([2, 4, 8, 16, 32])
        T = bs * nb
        L, top, K = rng.choice([8, 16, 32, 64, 128]), rng.choice([0, 1, 2, 3, 4]), rng.choice([1, 4, 5, 8, 16])
        if T > 2048 or L > T or top >= nb:
            continue
        strict, B = rng.random() < 0.5, rng.choice([1, 2, 3, 8])
        case = {"kind": "select", "seed": rng.randrange(1 << 30), "batch": B, "context": T, "blocks": nb,
                "buckets": rng.choice([8, 16]), "dtype": rng.choice(["bf16", "bf16", "fp32", "fp16"]),
                "quantize": rng.random() < 0.3}
        what = (bs, nb, L, top, K, strict, case)
        x = cases.make_inputs(case)
        xg = to_cuda(x)
        for t in sorted({0, 1, bs - 1, bs, rng.randrange(T), rng.randrange(T), T - 1}):
            got = relation_select_packed(*select_args(xg), position_tensor(t), L, top, K, strict)
            want = oracle.relation_select(*select_args(x), t, L, top, K, strict)
            assert _same_selection(got, want[:4]), ("decode form", what, t)
        # per-row form: random (sequence, position) rows with their own queries
        n = rng.choice([1, 5, 33])
        rb = torch.tensor([rng.randrange(B) for _ in range(n)], dtype=torch.int32)
        rp = torch.tensor([rng.randrange(T) for _ in range(n)], dtype=torch.int32)
        g = torch.Generator().manual_seed(case["seed"] + 1)
        queries = {k: torch.randn(n, w, generator=g).to(x["anchor_query"].dtype)
                   for k, w in (("anchor_query", 64), ("anchor_router_query", 64), ("partner_base", 128))}
        rows = [queries.get(k, x[k]) for k in SELECT_KEYS]
        got = relation_select_packed_rows(*[a.cuda() for a in rows], rb.cuda(), rp.cuda(), L, top, K, strict)
        per_sequence = {1, 3, 4, 8, 9, 10, 11}                    # caches and statistics: indexed by sequence
        for i in range(n):
            b = int(rb[i])
            one = [a[i:i + 1] if j in (0, 2, 7) else (a[b:b + 1] if j in per_sequence else a) for j, a in enumerate(rows)]
            want = oracle.relation_select(*one, int(rp[i]), L, top, K, strict)
            assert _same_selection(tuple(o[i:i + 1] for o in got), want[:4]), ("per-row form", what, i)
        # whole-sequence form against the per-row form it must equal bit for bit
        if L + top * bs <= 512 and T <= 256:
            g = torch.Generator().manual_seed(case["seed"] + 2)
            every = {k: torch.randn(B * T, w, generator=g).to(x["anchor_query"].dtype).cuda()
                     for k, w in (("anchor_query", 64), ("anchor_router_query", 64), ("partner_base", 128))}
            args = [every.get(k, xg[k]) for k in SELECT_KEYS]
            try:
                tiled = relation_select_packed_prefill(*args, T, L, top, K, strict)
            except (ValueError, RuntimeError) as error:          # shapes the tile form does not serve
                assert "shared memory" in str(error) or "support" in str(error), (what, error)
            else:
                rbp = torch.arange(B, dtype=torch.int32).repeat_interleave(T).cuda()
                rpp = torch.arange(T, dtype=torch.int32).repeat(B).cuda()
                assert _same_selection(tiled, relation_select_packed_rows(*args, rbp, rpp, L, top, K, strict)), \
                    ("whole-sequence form", what)
        done += 1
    assert_status_clear()


def test_random_reduce_and_router_configurations():
    from relation_lm.kernels.relation_reduce import (relation_hidden_cached, relation_norm_reduce,
                                                     relation_norm_reduce_rows)
    from relation_lm.kernels.router_cache import router_cache_update

    rng = random.Random(20262)
    for _ in range(100):
        g = torch.Generator().manual_seed(rng.randrange(1 << 30))
        name = rng.choice(["fp32", "bf16", "bf16", "fp16"])
        low, dtype = name != "fp32", DTYPES[name]
        B, K, T = rng.choice([1, 2, 3, 8, 40, 300]), rng.choice([1, 4, 5, 8]), rng.choice([16, 64, 256])
        R, H, d = rng.choice([64, 128]), rng.choice([256, 512, 1024, 2048, 2304]), rng.choice([128, 256, 512, 576, 768])
        what = (name, B, K, T, R, H, d)
        expanded = (torch.randn(B, T, 2 * H, generator=g) * 0.5).to(dtype)
        operand = torch.randn(B, T, R, generator=g).to(dtype)
        wm = (torch.randn(H, R, generator=g) * 0.05).to(dtype)
        ai = torch.randint(0, T, (B,), generator=g, dtype=torch.int32)
        pi = torch.randint(0, T, (B, K), generator=g, dtype=torch.int32)
        got = relation_hidden_cached(expanded.cuda(), operand.cuda(), ai.cuda(), pi.cuda(), wm.cuda())
        assert _close(got, oracle.relation_hidden(expanded, operand, ai, pi, wm)[0], low), ("relation hidden", what)

        raw = torch.randn(B, K, d, generator=g).to(dtype if low else torch.float32)
        scores = torch.randn(B, K, generator=g)
        if rng.random() < 0.5:
            scores[:, rng.randrange(K)] = -torch.inf
        if rng.random() < 0.2:
            scores[0] = -torch.inf                                  # a row without any active partner
        gamma, beta = torch.randn(d, generator=g) * 0.1 + 1.0, torch.randn(d, generator=g) * 0.1
        t = rng.randrange(T)
        got = relation_norm_reduce(raw.cuda(), scores.cuda(), gamma.cuda(), beta.cuda(), position_tensor(t), 1e-5)
        assert _close(got, oracle.relation_norm_reduce(raw.float(), scores, gamma, beta, t, 1e-5), low), ("norm-reduce", what, t)
        # per-row positions; thousands of rows take the warp-per-row kernel where it applies
        n = rng.choice([B, 2048 + 8 * rng.randrange(4)]) if d % 256 == 0 else B
        raw = torch.randn(n, K, d, generator=g).to(dtype if low else torch.float32)
        scores = torch.randn(n, K, generator=g)
        scores[::3, -1] = -torch.inf
        rp = torch.randint(0, T, (n,), generator=g, dtype=torch.int32)
        got = relation_norm_reduce_rows(raw.cuda(), scores.cuda(), gamma.cuda(), beta.cuda(), rp.cuda(), 1e-5)
        for i in range(0, n, max(1, n // 48)):
            want = oracle.relation_norm_reduce(raw[i:i + 1].float(), scores[i:i + 1], gamma, beta, int(rp[i]), 1e-5)
            assert _close(got[i:i + 1], want, low), ("norm-reduce rows", what, n, i)

        bs = rng.choice([8, 16, 32])
        Tr, Br = bs * rng.choice([2, 4, 8]), rng.choice([1, 3, 8])
        tt = rng.randrange(Tr)
        packed = torch.randn(Br, 512, generator=g).to(dtype)
        caches = [torch.randn(Br, Tr, 64, generator=g).to(dtype) for _ in range(4)]
        stats = [torch.randn(Br, Tr // bs, 4, 16, generator=g).to(dtype) for _ in range(4)]
        wa, wp = torch.randn(64, 3, generator=g) * 0.1, torch.randn(64, 3, generator=g) * 0.1
        mine = [c.cuda() for c in caches + stats]
        router_cache_update(packed[:, 384:448].cuda(), packed[:, 448:512].cuda(), *mine, wa.cuda(), wp.cuda(),
                            position_tensor(tt), bs)
        theirs = [c.float() for c in caches + stats]
        oracle.router_cache_update(packed[:, 384:448].float(), packed[:, 448:512].float(), *theirs, wa, wp, tt, bs,
                                   inplace=True, cache_dtype=dtype, stats_dtype=dtype)
        for a, b in zip(mine, theirs):
            assert torch.equal(a.float().cpu(), b), ("router update", name, bs, Tr, Br, tt)
    assert_status_clear()


def test_random_layer_tail_configurations():
    import test_gpu_layer_tail as tail
    from relation_lm.kernels.relation_reduce import relation_layer_tail_supported

    rng = random.Random(20263)
    done = 0
    while done < 300:
        dtype = rng.choice([torch.bfloat16, torch.float16])
        d, R = rng.choice([128, 256, 512]), rng.choice([64, 128, 192, 256])
        K = rng.choice([1, 2, 3, 4, 5, 7, 8, 16, 32])
        B, T = rng.choice([1, 2, 3, 4, 5, 7, 8, 9, 15, 16, 17, 31, 32, 33, 64]), rng.choice([8, 33, 96, 200])
        cluster = 4 * d // 128
        n_query = rng.choice([0, 16 * cluster, 32 * cluster, 256])
        t = rng.randrange(T)
        what = (str(dtype), B, K, d, R, T, n_query, t)
        if not relation_layer_tail_supported(B, K, R, 4 * d, d, n_query, dtype):
            continue
        x = tail._case(B, K, d, R, T, n_query, dtype, rng.randrange(1 << 30))
        if rng.random() < 0.3:
            x["scores"][:, rng.randrange(K)] = -torch.inf
        want_hidden, want_norm = tail._expected(x, t, dtype)
        hidden, normalized, query = tail._run(x, t, dtype)
        assert _close(hidden, want_hidden, True) and _close(normalized, want_norm, True), what
        if n_query:
            assert _close(query, oracle.linear(normalized.cpu(), x["wq"]), True), what
        again = tail._run(x, t, dtype)
        assert torch.equal(hidden, again[0]) and torch.equal(normalized, again[1]), what
        assert not n_query or torch.equal(query, again[2]), what
        done += 1
    assert_status_clear()


def test_random_decoder_configurations_match_cpu_port(monkeypatch):
    """fp32 decoders of random small configurations against the CPU port, position by position, sliding
    when the context is full.  Every selection is bit-equal to the oracle's on the selector's own inputs
    (indices and scores); the free-running port chooses the same rows at every layer and position and
    its logits agree to 2e-3 — until a near tie, if one comes up (the two sides' GEMMs sum in different
    orders, so their queries differ in the last bit): there the competing scores must agree to 1e-5 and
    the comparison of that configuration ends."""
    import relation_lm.inference.stateful_decode as decode_module
    from oracle.decode_port import OracleDecoder
    from relation_lm.inference.routed_model import RoutedRelationConfig, RoutedRelationLM

    calls = []
    plain_select = decode_module.relation_select_packed

    def recording_select(*args):
        out = plain_select(*args)
        calls.append((args[:14] + (args[14].clone(),) + args[15:], out))      # the position moves on after the step
        return out

    monkeypatch.setattr(decode_module, "relation_select_packed", recording_select)
    rng = random.Random(20264)
    near_ties = 0
    for _ in range(8):
        bs = rng.choice([4, 8, 16])
        nb = rng.choice([3, 4, 6, 8])
        T = bs * nb
        cfg = RoutedRelationConfig(
            vocab_size=300, boundary_vocab_size=8, d_model=rng.choice([128, 256]), layers=rng.choice([1, 2, 3]),
            max_context=T, block_size=bs, local_window=rng.choice([w for w in (4, 8, 16, 32) if w <= T]),
            top_blocks=rng.choice([t for t in (0, 1, 2, 3) if t < nb]), k_max=rng.choice([2, 4, 8]),
            relation_dim=rng.choice([64, 128]), strict_valid=rng.random() < 0.5)
        model = RoutedRelationLM(cfg, seed=rng.randrange(1000))
        B, steps = rng.choice([1, 2, 5]), T + 2 * bs + 3
        gpu = decode_module.StatefulDecoder(model, B, "cuda", torch.float32)
        cpu = OracleDecoder(model, B, torch.float32)
        g = torch.Generator().manual_seed(rng.randrange(1 << 30))
        tokens = torch.randint(0, 300, (B, steps), generator=g)
        bounds = torch.randint(0, 8, (B, steps), generator=g)
        in_step, position = True, 0
        for t in range(steps):
            if position == T:
                gpu.slide(1)
                if in_step:
                    cpu.slide(1)
                position -= bs
            position += 1
            calls.clear()
            tl, _ = gpu.step(tokens[:, t].cuda(), bounds[:, t].cuda(), keep_selection=True)
            assert len(calls) == cfg.layers
            for layer, (args, out) in enumerate(calls):
                host = [a.cpu() if isinstance(a, torch.Tensor) else a for a in args]
                want = oracle.relation_select(*host[:14], int(host[14]), *host[15:])
                assert _same_selection(out, want[:4]), ("selector on its own inputs", cfg, t, layer)
            if not in_step:
                continue
            ctl, _ = cpu.step(tokens[:, t], bounds[:, t])
            for layer, ((ga, gp), (ca, cp)) in enumerate(zip(gpu.last_selection, cpu.last_selection)):
                if torch.equal(ga.cpu(), ca) and torch.equal(gp.cpu(), cp):
                    continue
                # a different row on the two sides: only where the rows' scores tie to rounding, judged
                # on the selector's own inputs (gate scores are plain 64-wide dot products)
                host = [a.cpu() if isinstance(a, torch.Tensor) else a for a in calls[layer][0]]
                mine = [o.cpu() for o in calls[layer][1]]
                for b in range(B):
                    if int(ga[b]) != int(ca[b]):
                        other = float(host[0][b].double() @ host[1][b, int(ca[b])].double()) / 8.0       # gate width 64
                        assert abs(other - float(mine[1][b])) <= 1e-5 * max(1.0, abs(other)), (cfg, t, layer, b)
                        continue                              # another anchor: other partner queries
                    query = host[7][b, :64].double() + host[8][b, int(ga[b]), :64].double()
                    kept = mine[3][b][torch.isfinite(mine[3][b])]
                    for p in set(cp[b].tolist()) - set(gp[b].cpu().tolist()):
                        other = float(query @ host[9][b, p].double()) / 8.0
                        assert kept.numel() and abs(other - float(kept.min())) <= 1e-5 * max(1.0, abs(other)), (cfg, t, layer, b, p)
                near_ties += 1
                in_step = False
                break
            if in_step:
                assert torch.allclose(tl.cpu(), ctl, atol=2e-3, rtol=1e-4), (cfg, t)
    assert near_ties <= 2, near_ties
    assert_status_clear()


def test_random_multi_anchor_configurations():
    """Routed multi-anchor selection in random shapes: the one-launch per-row form against the oracle's
    slot-by-slot composition (anchors, activity, partner indices and scores bit-exact), and the
    whole-sequence tile form against the per-row form, bit for bit."""
    from relation_lm.kernels.multi_select import relation_select_multi_prefill, relation_select_multi_rows

    rng = random.Random(20265)
    done = 0
    while done < 40:
        S, B = rng.choice([1, 2, 3, 4, 8]), rng.choice([1, 2, 3])
        bs, NB = rng.choice([8, 16, 32, 64]), rng.choice([2, 4, 8, 16])
        T = bs * NB
        L, top, K = rng.choice([8, 16, 32, 64, 128]), rng.choice([0, 1, 2, 3]), rng.choice([1, 2, 4, 8])
        if T > 512 or L > T or top >= NB:
            continue
        strict = rng.random() < 0.5
        dt = rng.choice([torch.bfloat16, torch.bfloat16, torch.float16, torch.float32])
        what = (S, B, T, NB, L, top, K, strict, dt)
        g = torch.Generator().manual_seed(rng.randrange(1 << 30))
        N = B * T
        rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
        x = [rn(N, S, 64).to(dt), rn(S, B, T, 64).to(dt), rn(N, S, 64).to(dt), rn(S, B, NB, 4, 16).to(dt),
             rn(S, B, NB, 4, 16).abs().to(dt), rn(S, 4), rn(S, 4, 16), rn(N, S, 128).to(dt), rn(S, B, T, 128).to(dt),
             rn(S, B, T, 64).to(dt), rn(S, B, NB, 4, 16).to(dt), rn(S, B, NB, 4, 16).abs().to(dt), rn(S, 4), rn(S, 4, 16)]
        if rng.random() < 0.5:                                  # exact duplicates: ties between positions and slots
            x[1][0, :, 5::7] = x[1][0, :, 4:5]
            x[9][0, :, 3::5] = x[9][0, :, 2:3]
        aq, ak, arq, am, as_, ag, ab, pb, pac, pk, pm, ps, pg, pbias = x
        row_batch = torch.arange(B, dtype=torch.int32).repeat_interleave(T)
        row_pos = torch.arange(T, dtype=torch.int32).repeat(B)
        d = [v.cuda() for v in x]
        got = relation_select_multi_rows(*d, row_batch.cuda(), row_pos.cuda(), L, top, K, strict)
        active = torch.arange(S)[None, :] <= row_pos[:, None]
        taken = torch.full((N, S), -1, dtype=torch.int32)
        anchors = torch.zeros(N, S, dtype=torch.int32)
        for s in range(S):
            idx, score = oracle.anchor_select(aq[:, s], ak[s], arq[:, s], am[s], as_[s], ag[s], ab[s], 0, L, top, strict,
                                              row_batch=row_batch, row_pos=row_pos, exclude_index=taken.clone())
            live = active[:, s] & torch.isfinite(score)
            anchors[:, s] = torch.where(live, idx, torch.zeros_like(idx))
            taken[:, s] = torch.where(live, idx, torch.full_like(idx, -1))
            active[:, s] = live
        assert torch.equal(got[0].cpu(), anchors), what
        assert torch.equal(got[2].cpu(), active), what
        for s in range(S):
            v = pb[:, s].float() + pac[s][row_batch.long(), anchors[:, s].long()].float()
            idx, score = oracle.partner_topk(v[:, :64], pk[s], v[:, 64:], pm[s], ps[s], pg[s], pbias[s], 0, taken[:, s],
                                             L, top, K, strict, row_batch=row_batch, row_pos=row_pos, exclude_index=taken)
            live = active[:, s, None] & torch.isfinite(score)
            assert torch.equal(got[5].cpu()[:, s], live), (what, s)
            assert torch.equal(got[3].cpu()[:, s][live], idx[live]), (what, s)
            assert torch.equal(got[4].cpu()[:, s][live], score[live]), (what, s)
        if dt == torch.bfloat16 and L + top * bs <= 512:            # the tile form serves bfloat16
            try:
                tiled = relation_select_multi_prefill(*d, T, L, top, K, strict)
            except (ValueError, RuntimeError) as error:
                assert "shared memory" in str(error) or "support" in str(error), (what, error)
            else:
                for a, b in zip(tiled, got):
                    same = torch.equal(a.view(torch.int32), b.view(torch.int32)) if a.dtype == torch.float32 else torch.equal(a, b)
                    assert same, ("whole-sequence form", what)
        done += 1
    assert_status_clear()
