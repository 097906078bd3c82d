"""The Lomopel decoder in the engine against the plain implementation (tests/plain/lomopel_plain.py):
small configurations made here, random weights, float32 and bfloat16. Each mechanism alone (the
kernels on inputs made so that a fault shows: one key far back, at a page's border, just inside and
just outside the window, a sink that outweighs the keys; and models of one layer), whole prompts
against tokens one by one, portions down to two tokens, unequal requests side by side against each
alone, pages and state slots that are given back and used again, long decoding, and greedy
generation through `LLM` and the command line."""
import json
import os
import random

import pytest
import torch

from tests.plain import lomopel_plain as plain
from tests.util import max_rel_diff

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _configs():
    from vllm_oxide_b200.config import GatedDeltaConfig as GD, LomopelConfig, LomopelLayer as L, SoftmaxMixerConfig as SM
    att = SM(heads=4, kv_heads=2, dim=24, vdim=40, scale=0.2, q_temp=(0.5, 7), v_mix=True)
    att_mix = SM(heads=2, kv_heads=2, dim=16, vdim=40, scale=0.3, v_mix=True)                    # no query factor
    att_plain = SM(heads=1, kv_heads=1, dim=10, vdim=6, scale=0.35, q_temp=(0.25, 1))           # every 1; sizes no vector load takes
    left = SM(heads=4, kv_heads=1, dim=32, vdim=16, scale=0.3, window=9, rot_dims=16, rot_base=100.0)
    left_full = SM(heads=2, kv_heads=2, dim=16, vdim=16, scale=0.25, window=16, rot_dims=16, rot_base=10000.0)    # all of a head rotated
    left_one = SM(heads=3, kv_heads=3, dim=10, vdim=6, scale=0.4, window=1, rot_dims=4, rot_base=50.0)            # sees itself only
    left_wide = SM(heads=2, kv_heads=1, dim=8, vdim=24, scale=0.5, window=200)                                    # no rotation, a window never reached
    # keys and values of one size, 64 or 128: in bfloat16 these take the framework's tensor-core attention kernels;
    # a window that is no multiple of a tile of keys
    left_tc = SM(heads=6, kv_heads=2, dim=64, vdim=64, scale=0.2, window=37, rot_dims=8, rot_base=1000.0)
    att_tc = SM(heads=4, kv_heads=1, dim=64, vdim=64, scale=0.04, q_temp=(0.3, 16), v_mix=True)
    att_tc128 = SM(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.03)
    right = GD(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, decay_rank=5, gate_rank=6)
    right_wide = GD(heads=2, kv_heads=2, dim=40, vdim=8, conv=4, decay_rank=3, gate_rank=3)
    right_one = GD(heads=3, kv_heads=1, dim=8, vdim=12, conv=1, decay_rank=2, gate_rank=7)       # no convolution state at all
    right_five = GD(heads=1, kv_heads=1, dim=24, vdim=16, conv=5, decay_rank=4, gate_rank=4)
    par = L("parallel", left=left, right=right, left_scale=0.7, right_scale=1.3, ff=0)
    return {
        "A": LomopelConfig(vocab=97, width=64, embedding_scale=3.7, norm_eps=1e-5, layers=(
            L("attention", attention=att, ff=96), par, L("attention", attention=att_mix, ff=80),
            L("parallel", left=left_full, right=right_wide, left_scale=1.1, right_scale=0.6, ff=72))),
        # a width that is no multiple of 4 or 8, a parallel layer first, no layer mixes values, the last layer without feed-forward
        "B": LomopelConfig(vocab=131, width=42, embedding_scale=1.0, norm_eps=1e-6, layers=(
            L("parallel", left=left_one, right=right_one, left_scale=1.0, right_scale=1.0, ff=56),
            L("attention", attention=att_plain, ff=0),
            L("parallel", left=left_wide, right=right_five, left_scale=0.5, right_scale=2.0, ff=0))),
        # sizes that take the tensor-core kernels in bfloat16; three layers mix values
        "T": LomopelConfig(vocab=77, width=96, embedding_scale=2.0, norm_eps=1e-5, layers=(
            L("attention", attention=att_tc, ff=64), L("parallel", left=left_tc, right=right, left_scale=1.2, right_scale=0.9, ff=64),
            L("attention", attention=att_tc, ff=0), L("attention", attention=att_tc128, ff=64))),
        "attention": LomopelConfig(vocab=50, width=48, embedding_scale=2.5, norm_eps=1e-5, layers=(L("attention", attention=att, ff=0),)),
        "parallel": LomopelConfig(vocab=50, width=48, embedding_scale=2.5, norm_eps=1e-5, layers=(par,)),
    }


def _model_dir(tmp_path, name, seed=11):
    from vllm_oxide_b200.weights import write_random_model
    d = os.path.join(str(tmp_path), f"lomopel_{name}_{seed}")
    if not os.path.exists(os.path.join(d, "model.safetensors")):
        write_random_model(d, _configs()[name], seed, std=0.25, norm_jitter=0.3)
    return d


def _plain_logits(model_dir, tokens):
    from safetensors.torch import load_file
    cfg = json.load(open(os.path.join(model_dir, "config.json")))
    return plain.forward(cfg, load_file(os.path.join(model_dir, "model.safetensors")), tokens, torch.float64)


def _runner(model_dir, dtype, page=8, pages=24, max_seqs=3, rows=192):
    from vllm_oxide_b200.config import EngineConfig
    from vllm_oxide_b200.engine import ModelRunner
    eng = EngineConfig(max_batch_tokens=rows, max_seqs=max_seqs, max_model_len=page * pages, block_size=page, num_pages=pages,
                       dtype=dtype, cuda_graphs=False)
    return ModelRunner.from_dir(model_dir, eng)


def _tokens(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


# float32: the engine against float64, rounding over a few hundred operations per logit. bfloat16: the projections'
# inputs and outputs, the cache and the gated results are rounded to 8 mantissa bits (2^-9 relative each), a dozen
# roundings a layer over up to four layers.
TOL = {"float32": 3e-5, "bfloat16": 6e-2}


def _close(got, want, dtype) -> bool:
    """float32: every logit within TOL of the largest. bfloat16: the typical row tight (root mean square of a row's
    error against that of its logits, averaged over the rows) and no logit anywhere off by more than a tenth of the
    largest. A key that is skipped, a wrong page, a window one token off or a lost state moves rows by far more."""
    if dtype == "float32":
        return max_rel_diff(got, want) < TOL[dtype]
    err = (got.double() - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()
    return float(err.mean()) < 2.5e-2 and max_rel_diff(got, want) < 0.1


def _poison(runner):
    """Whatever lies in pages that nobody holds must never be read."""
    for ts in runner.pools.kv.values():
        for t in ts:
            t.fill_(float("nan"))


def _replay(session, reqs, schedule, first_step=0):
    """schedule: a list of steps, each a list of (name, count). Returns {name: logits of all its tokens}."""
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    for n, step in enumerate(schedule):
        entries, end = [], []
        for name, count in step:
            lo = at[name]
            entries.append({"id": name, "tokens": reqs[name][lo:lo + count], "want": list(range(count))})
            at[name] = lo + count
            if at[name] == len(reqs[name]):
                end.append(name)
        out = session.run_step({"step": first_step + n, "entries": entries, "end": end})
        r = 0
        for name, count in step:
            got[name].append(out[r:r + count])
            r += count
    return {k: torch.cat(v) for k, v in got.items() if v}


# ------------------------------------------------------------------------------------ small kernels
def test_scaled_embedding_scaled_add_and_gelu_gate():
    from vllm_oxide_b200 import kernels
    torch.manual_seed(0)
    table = torch.randn(20, 42, device=DEV).bfloat16()
    toks = torch.tensor([3, 19, 0], dtype=torch.int32, device=DEV)
    out = torch.empty(3, 42, device=DEV)
    kernels.embed(table, toks, out, None, 2.75)
    assert torch.equal(out, table[toks.long()].float() * 2.75)
    for h in (42, 64):                                   # the plain kernel and the 16-byte one
        resid, delta = torch.randn(5, h, device=DEV), torch.randn(5, h, device=DEV).bfloat16()
        w, sc = torch.randn(h, device=DEV), torch.randn(h, device=DEV)
        want_resid = resid.double() + delta.double() * sc.double()
        want = plain.rms(want_resid, 1e-5) * w.double()
        normed = torch.empty(5, h, device=DEV)
        kernels.add_rmsnorm(resid, delta, w, 1e-5, normed, None, sc)
        assert max_rel_diff(resid, want_resid) < 1e-6 and max_rel_diff(normed, want) < 1e-5
        rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
        picked = torch.empty(2, h, device=DEV)
        before = resid.clone()
        kernels.add_rmsnorm(resid, delta, w, 1e-5, picked, rows, sc)       # looked at only: the residual stays
        assert torch.equal(resid, before)
        assert max_rel_diff(picked, (plain.rms(before.double() + delta.double() * sc.double(), 1e-5) * w.double())[[4, 1]]) < 1e-5
    for cols in (30, 64):
        gu = torch.randn(4, 2 * cols, device=DEV) * 3
        act = torch.empty(4, cols, device=DEV)
        kernels.glu(gu, act, "gelu_tanh")
        assert max_rel_diff(act, plain.gelu_tanh(gu[:, :cols].double()) * gu[:, cols:].double()) < 1e-6
    a, w, b = torch.randn(7, 33, device=DEV), torch.randn(19, 33, device=DEV), torch.randn(19, device=DEV)
    out = torch.empty(7, 19, device=DEV)
    kernels.linear(a, w, out, b)
    assert max_rel_diff(out, a.double() @ w.double().T + b.double()) < 1e-6
    out16 = torch.empty(7, 19, device=DEV, dtype=torch.bfloat16)
    kernels.linear(a.bfloat16(), w.bfloat16(), out16, b.bfloat16())
    assert max_rel_diff(out16, a.bfloat16().double() @ w.bfloat16().double().T + b.bfloat16().double()) < 1e-2


@pytest.mark.parametrize("rows", [8, 40, 700])
def test_products_whose_epilogue_applies_the_gelu_gate(rows):
    """Few rows: the one-SM tcgen05 product; many: the two-SM one. Both against gate and up done plainly."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(2)
    K, I = 96, 136
    x = (torch.randn(rows, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV) * 0.3).bfloat16()
    want = plain.gelu_tanh(x.double() @ w[:I].double().T) * (x.double() @ w[I:].double().T)
    out = torch.empty(rows, I, dtype=torch.bfloat16, device=DEV)
    if rows <= kernels.FUSED_GEMM_MAX_ROWS:
        kernels.gemm_swiglu(x, w, out, activation="gelu_tanh")
    else:
        kernels.gemm_pair_swiglu(x, w, out, "gelu_tanh")
    kernels.gemm_sm100_check()
    assert max_rel_diff(out, want) < 1e-2


# ------------------------------------------------------------------------------------ attention kernels
def _paged(total, page, heads_widths, dtype, spare=3):
    """Block tables over scattered pages for requests of `total` tokens; cache tensors full of NaN."""
    pages_per = [-(-t // page) for t in total]
    n = sum(pages_per) + spare
    perm = torch.randperm(n)
    tables = torch.full((len(total), max(pages_per) + 2), -1, dtype=torch.int32)
    at = 0
    for s, pp in enumerate(pages_per):
        tables[s, :pp] = perm[at:at + pp].to(torch.int32)
        at += pp
    caches = [torch.full((n, h, page, w), float("nan"), dtype=dtype, device=DEV) for h, w in heads_widths]
    return tables, caches


def _fill(cache, tables, s, x, page):
    """x [tokens, heads, width] of request s into its pages."""
    idx = torch.arange(x.shape[0])
    pg, off = tables[s, idx // page].long(), idx % page
    cache[pg.to(DEV), :, off.to(DEV)] = x.to(device=DEV, dtype=cache.dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,DV,window,sink,gate", [
    (4, 2, 24, 40, 0, True, False), (3, 3, 10, 6, 5, False, True), (8, 4, 64, 64, 45, False, True), (6, 3, 80, 56, 0, True, False),
    (6, 2, 32, 48, 37, True, True), (2, 1, 128, 16, 1, False, False), (8, 2, 64, 64, 0, True, False), (4, 2, 128, 128, 0, True, True),
    (4, 1, 128, 128, 100, False, False)])
def test_attention_kernels_far_key_page_borders_window_edges_and_sink(dtype, H, G, D, DV, window, sink, gate):
    """Two requests in one batch over scattered pages, one with a context in the cache and a portion of
    rows, one a single decoded token far into its context. Queries and keys are made so that single
    keys outweigh all others: one far back (position 3), one at a page's last slot, the one just
    inside the window and, with a weight that would swamp everything if it were seen, the one just
    outside. The sink of one head outweighs every key."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(7)
    page, scale = 8, 0.3
    ctxs, lens = (150, 320), (70, 1)
    total = [c + n for c, n in zip(ctxs, lens)]
    tables, (kc, vc) = _paged(total, page, [(G, D), (G, DV)], dtype)
    k = [torch.randn(t, G, D) * 0.5 for t in total]
    v = [torch.randn(t, G, DV) for t in total]
    T = sum(lens)
    q = torch.randn(T, H, D) * 0.5
    group = H // G

    def aim(row, s, pos_key, weight):
        for a in range(H):
            kk = k[s][pos_key, a // group]
            q[row, a] = weight * kk / kk.norm() ** 2 / scale
    far_row = 60                                         # request 0, position 210
    if window == 0:
        aim(far_row, 0, 3, 12.0)
        aim(T - 1, 1, 7, 12.0)                           # the decoded token looks at a page's last slot, 313 back
    else:
        pos = ctxs[0] + far_row
        if window > 1:
            aim(far_row, 0, pos - window + 1, 12.0)      # just inside
        # a key just outside that would dominate everything: its score is larger than any other
        k[0][pos - window] = 30.0 * q[far_row, 0] / q[far_row, 0].norm() ** 2 / scale
        pos1 = total[1] - 1
        k[1][pos1 - window] = 30.0 * q[T - 1, 0] / q[T - 1, 0].norm() ** 2 / scale
    for s in range(2):
        _fill(kc, tables, s, k[s], page)
        _fill(vc, tables, s, v[s], page)
    sk = torch.randn(H) if sink else None
    if sink:
        sk[1] = 25.0                                     # head 1's result all but vanishes
    g = torch.randn(T, H * DV) if gate else None
    positions = torch.cat([torch.arange(ctxs[s], total[s]) for s in range(2)]).to(device=DEV, dtype=torch.int32)
    row_seq = torch.cat([torch.full((lens[s],), s) for s in range(2)]).to(device=DEV, dtype=torch.int32)
    qd = q.reshape(T, H * D).to(device=DEV, dtype=dtype)
    gd = g.to(device=DEV, dtype=dtype) if gate else None
    wide = torch.full((T, H * DV + 8), float("nan"), dtype=dtype, device=DEV)
    out = wide[:, 8:]                                    # a column range of a wider buffer
    kernels.flex_attention(qd, out, kc, vc, tables.to(DEV), row_seq, positions, H, G, D, DV, scale, window,
                           sk.to(DEV) if sink else None, gd, 0.75)
    r0 = 0
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    wants = []
    for s in range(2):
        kk, vv = k[s].to(dtype).double(), v[s].to(dtype).double()
        qq = qd[r0:r0 + lens[s]].cpu().double().reshape(lens[s], H, D)
        i, j = torch.arange(ctxs[s], total[s])[:, None], torch.arange(total[s])[None, :]
        visible = (j <= i) & ((i - j < window) if window else torch.ones_like(j <= i))
        kx, vx = kk.repeat_interleave(group, 1), vv.repeat_interleave(group, 1)
        w = plain.softmax_rows(torch.einsum("ihd,jhd->hij", qq, kx) * scale, visible, sk.double() if sink else None)
        want = torch.einsum("hij,jhd->ihd", w, vx).reshape(lens[s], H * DV) * 0.75
        if gate:
            want = want * torch.sigmoid(gd[r0:r0 + lens[s]].cpu().double())
        assert max_rel_diff(out[r0:r0 + lens[s]].cpu(), want) < tol, s
        wants.append(want)
        if s == 0 and window == 0:
            assert float(w[0, far_row, 3]) > 0.5         # the far key is what the row is made of
        if s == 0 and window > 1:
            assert float(w[0, far_row, ctxs[0] + far_row - window + 1]) > 0.5
        if sink and s == 0:
            assert float(w[1].sum(-1).max()) < 1e-3      # the sink took it all
        r0 += lens[s]
    assert bool(torch.isnan(wide[:, :8]).all())
    if dtype != torch.bfloat16:
        return
    # the same rows through the tensor-core kernels, which end with the same sink, gate and factor
    want = torch.cat(wants)
    starts = torch.tensor([0, lens[0], T], dtype=torch.int32, device=DEV)
    ctxd = torch.tensor(ctxs, dtype=torch.int32, device=DEV)
    skd = sk.to(DEV) if sink else None
    assert kernels.attn_prefill_mma_any_supported(H, G, D, DV, page) == (D % 8 == 0 and DV % 8 == 0)
    if kernels.attn_prefill_mma_any_supported(H, G, D, DV, page):
        # keys and values of sizes of their own, in tiles padded with zero columns
        out.fill_(float("nan"))
        kernels.attn_prefill_mma_any(qd, out, kc, vc, tables.to(DEV), starts, ctxd, 2, lens[0], H, G, D, DV, scale, window, skd, gd, 0.75)
        assert max_rel_diff(out.cpu(), want) < tol
        assert bool(torch.isnan(wide[:, :8]).all())
    if D != DV or D not in kernels.TENSOR_CORE_HEAD_DIMS:
        return
    out.fill_(float("nan"))
    kernels.attn_prefill_mma(qd, out, kc, vc, tables.to(DEV), starts, ctxd, 2, lens[0], H, G, D, scale, window, skd, gd, 0.75)
    assert max_rel_diff(out.cpu(), want) < tol
    if window == 0 and not gate:
        plain_out = torch.full((T, H * DV), float("nan"), dtype=dtype, device=DEV)
        kernels.attn_prefill_sm100(qd, plain_out, kc, vc, tables.to(DEV), starts, ctxd, 2, lens[0], H, G, D, scale, skd)
        assert max_rel_diff(plain_out.cpu(), want / 0.75) < tol
    for splits, wide_merge in ((1, False), (4, False), (8, False), (12, True)):
        one = torch.full((1, H * DV + 8), float("nan"), dtype=dtype, device=DEV)
        partials = torch.empty(kernels.attn_decode_partial_floats(1, G, D, splits), device=DEV) if wide_merge else None
        arrived = torch.zeros(G, dtype=torch.int32, device=DEV) if wide_merge else None
        kernels.attn_decode_mma(qd[T - 1:], one[:, 8:], kc, vc, tables[1:].to(DEV).contiguous(), positions[T - 1:].contiguous(), H, G, D, scale,
                                window, splits, partials, arrived, skd, gd[T - 1:] if gate else None, 0.75)
        assert max_rel_diff(one[:, 8:].cpu(), want[T - 1:]) < tol, splits


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_preparation_rotation_norm_factor_mixing_and_cache_write(dtype):
    from vllm_oxide_b200 import kernels
    from vllm_oxide_b200.parts.rotary import rotary_inv_freq
    torch.manual_seed(3)
    H, G, D, DV, page, T = 3, 1, 20, 12, 4, 9
    rot, base, eps = 8, 50.0, 1e-5
    proj = (torch.randn(T, 5 + H * D + G * D + G * DV)).to(dtype)
    pos = torch.tensor([0, 1, 2, 3, 126, 127, 128, 1023, -1], dtype=torch.int32)
    slots = torch.tensor([5, 6, 7, 0, 17, 18, 19, 2, -1], dtype=torch.int32)
    kc = torch.full((6, G, page, D), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full((6, G, page, DV), float("nan"), dtype=dtype, device=DEV)
    qo = torch.zeros(T, H * D, dtype=dtype, device=DEV)
    inv = torch.from_numpy(rotary_inv_freq(rot, base).copy()).to(DEV)
    first = torch.randn(T, G * DV).to(dtype)
    lam = torch.tensor([0.3], device=DEV)
    kernels.flex_prep(proj.to(DEV), 5, 5 + H * D, 5 + H * D + G * D, pos.to(DEV), slots.to(DEV), inv, rot, True, eps, (0.4, 128),
                      lam, first.to(DEV), 2, qo, kc, vc, H, G, D, DV)
    p64 = proj.double()

    def rotated(x, heads):
        out = torch.empty(T, heads, D, dtype=torch.float64)
        for t in range(T):
            z = plain.rotate_partial(x[t].reshape(1, heads, D).repeat(max(int(pos[t]), 0) + 1, 1, 1), rot, base)
            out[t] = z[max(int(pos[t]), 0)]
        return plain.rms(out, eps)
    q = rotated(p64[:, 5:5 + H * D], H)
    fac = 1.0 + 0.4 * torch.log((torch.div(pos.clamp(min=0) + 1, 128, rounding_mode="floor") + 1).double())
    q = q * fac[:, None, None]
    k = rotated(p64[:, 5 + H * D:5 + H * D + G * D], G)
    v = 0.7 * p64[:, -G * DV:] + 0.3 * first.double()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert max_rel_diff(qo[:8].cpu(), q[:8].reshape(8, H * D)) < tol
    assert bool((qo[8] == 0).all())                       # the padding row is left alone
    for t in range(8):
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        assert max_rel_diff(kc[pg, :, off].cpu(), k[t]) < tol and max_rel_diff(vc[pg, :, off].cpu(), v[t].reshape(G, DV)) < tol
    written = {int(s) for s in slots[:8]}
    for sl in range(6 * page):
        if sl not in written:
            assert bool(torch.isnan(kc[sl // page, :, sl % page]).all())
    # the first mixing layer leaves its values, unmixed, for the others
    left = torch.zeros(T, G * DV, dtype=dtype, device=DEV)
    kernels.flex_prep(proj.to(DEV), 5, 5 + H * D, 5 + H * D + G * D, pos.to(DEV), None, None, 0, False, 0.0, None, None, left, 1, qo, kc, vc,
                      H, G, D, DV)
    assert torch.equal(left[:8].cpu(), proj[:8, -G * DV:]) and torch.equal(qo[:8].cpu(), proj[:8, 5:5 + H * D])


# ------------------------------------------------------------------------------------ gated delta rule kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,K,V,taps", [(4, 2, 16, 24, 3), (2, 2, 40, 8, 4), (3, 1, 8, 12, 1), (1, 1, 136, 16, 5), (2, 1, 264, 8, 2)])
def test_gated_delta_kernels_portions_state_and_shared_heads(dtype, H, G, K, V, taps):
    """Preparation, convolution state and scan over two requests cut into portions of 1, 2, 3 and more tokens
    (shorter than the convolution, too), in slots that are not their order, against the whole sequences done
    plainly; then the slots are zeroed and used again."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(5)
    C, ra = 2 * G * K + H * V, 3
    n = (23, 9)
    x = [(torch.randn(t, C + H + 2)).to(dtype) for t in n]                  # q | k | v | strengths | 2 spare columns
    low = [(torch.randn(t, 4 + H * K) * 2).to(dtype) for t in n]
    cw = torch.randn(C, taps) * 0.5
    a_log, dt_bias = torch.randn(H) * 0.5 - 1.0, torch.randn(H * K)

    def want(s):
        xs, ls = x[s].double(), low[s].double()
        t = n[s]
        q = plain.causal_conv_silu(xs[:, :G * K], cw[:G * K].double()).reshape(t, G, K)
        k = plain.causal_conv_silu(xs[:, G * K:2 * G * K], cw[G * K:2 * G * K].double()).reshape(t, G, K)
        v = plain.causal_conv_silu(xs[:, 2 * G * K:C], cw[2 * G * K:].double()).reshape(t, H, V).to(dtype).double()
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * K ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        q, k = q.repeat_interleave(H // G, 1), k.repeat_interleave(H // G, 1)
        beta = torch.sigmoid(xs[:, C:C + H])
        g = torch.exp(-torch.exp(a_log.double())[None, :, None] * torch.nn.functional.softplus(ls[:, 4:] + dt_bias.double()).reshape(t, H, K))
        S = torch.zeros(H, K, V, dtype=torch.float64)
        o = torch.zeros(t, H, V, dtype=torch.float64)
        for i in range(t):
            S = g[i][:, :, None] * S
            u = beta[i][:, None] * (v[i] - torch.einsum("hkv,hk->hv", S, k[i]))
            S = S + k[i][:, :, None] * u[:, None, :]
            o[i] = torch.einsum("hkv,hk->hv", S, q[i])
        return o.reshape(t, H * V), S
    state = torch.full((4, H, K, V), float("nan"), device=DEV)
    cstate = torch.full((4, max(taps - 1, 0), C), float("nan"), device=DEV) if taps > 1 else None
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for slots in ((2, 0), (1, 2)):                       # the second round reuses slot 2 for the other request
        for sl in slots:
            state[sl].zero_()
            if cstate is not None:
                cstate[sl].zero_()
        cuts = [[(0, 2), (1, 1)], [(0, 1), (1, 3)], [(1, 2)], [(0, 3), (1, 1)], [(0, 1)], [(0, 16), (1, 2)]]
        at, got = [0, 0], [[], []]
        for step in cuts:
            rows = torch.cat([x[s][at[s]:at[s] + c] for s, c in step]).to(DEV)
            lows = torch.cat([low[s][at[s]:at[s] + c] for s, c in step]).to(DEV)
            T = rows.shape[0]
            starts = torch.tensor([0] + torch.tensor([c for _, c in step]).cumsum(0).tolist(), dtype=torch.int32, device=DEV)
            rs = torch.cat([torch.full((c,), i) for i, (_, c) in enumerate(step)]).to(device=DEV, dtype=torch.int32)
            pos = torch.cat([torch.arange(at[s], at[s] + c) for s, c in step]).to(device=DEV, dtype=torch.int32)
            sl = torch.tensor([slots[s] for s, _ in step], dtype=torch.int32, device=DEV)
            q, k = torch.empty(T, G * K, device=DEV), torch.empty(T, G * K, device=DEV)
            v = torch.empty(T, H * V, dtype=dtype, device=DEV)
            decay, beta, o = torch.empty(T, H * K, device=DEV), torch.empty(T, H, device=DEV), torch.empty(T, H * V, device=DEV)
            kernels.gated_delta_prep(rows, 0, C, lows, 4, cw.to(DEV), cstate, a_log.to(DEV), dt_bias.to(DEV), pos, rs, starts, sl, len(step),
                                     H, G, K, V, q, k, v, decay, beta)
            # the convolution state is moved on by a kernel of its own, or by the scan on its way
            if cstate is not None and slots == (2, 0):
                kernels.conv_state_update(rows, 0, cstate, starts, sl, len(step))
            kernels.recurrence_scan(2, q, k, v, decay, beta, None, state, starts, sl, len(step), H, o, rk_heads=G,
                                    conv_x=rows[:, :C] if cstate is not None and slots != (2, 0) else None,
                                    conv_state=cstate if slots != (2, 0) else None)
            r = 0
            for s, c in step:
                got[s].append(o[r:r + c].cpu())
                at[s] += c
                r += c
        for s in range(2):
            o_want, S_want = want(s)
            assert at[s] == n[s]
            assert max_rel_diff(torch.cat(got[s]), o_want) < tol, (slots, s)
            assert max_rel_diff(state[slots[s]].cpu(), S_want) < tol
    assert bool(torch.isnan(state[3]).all())              # a slot nobody held was never touched


def test_gated_delta_post_norm_gate_scale_into_a_column_range():
    from vllm_oxide_b200 import kernels
    torch.manual_seed(1)
    T, H, V = 5, 3, 20
    o, gate, w = torch.randn(T, H * V, device=DEV), torch.randn(T, H * V + 4, device=DEV), torch.randn(V, device=DEV)
    wide = torch.full((T, 7 + H * V), float("nan"), device=DEV)
    kernels.recurrence_post(o, gate[:, 4:], w.repeat(H).contiguous(), "sigmoid", 1e-5, H, wide[:, 7:], 1.3)
    want = plain.rms(o.double().reshape(T, H, V), 1e-5) * w.double() * torch.sigmoid(gate[:, 4:].double()).reshape(T, H, V) * 1.3
    assert max_rel_diff(wide[:, 7:], want.reshape(T, H * V)) < 1e-5 and bool(torch.isnan(wide[:, :7]).all())


# ------------------------------------------------------------------------------------ models in the engine
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention", "parallel"])
def test_each_mixer_alone_whole_prompt_and_token_by_token(tmp_path, name, dtype):
    from vllm_oxide_b200.replay.trace import TraceSession
    d = _model_dir(tmp_path, name)
    toks = _tokens(45, 50, 5)
    want = _plain_logits(d, toks)
    runner = _runner(d, dtype)
    _poison(runner)
    s = TraceSession(runner)
    whole = _replay(s, {"a": toks}, [[("a", 45)]])["a"]
    assert _close(whole, want, dtype)
    # most of it at once, the rest one by one, in the slot and the pages that were just given back
    _poison(runner)
    single = _replay(s, {"b": toks}, [[("b", 19)]] + [[("b", 1)]] * 26, first_step=10)["b"]
    assert _close(single, want, dtype)
    if dtype == "float32":
        assert max_rel_diff(single, whole) < 3e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "T"])
def test_portions_unequal_batches_and_reuse(tmp_path, name, dtype):
    """Four requests of unequal length in a pool that cannot hold them all at once: portions from 2
    tokens up beside single tokens, portions that end inside a page and inside a window, a request
    that sits out a step, a fourth request that takes over a slot and pages that were given back in
    the middle. Every row equals the plain model's."""
    from vllm_oxide_b200.replay.trace import TraceSession
    d = _model_dir(tmp_path, name)
    vocab = _configs()[name].vocab
    reqs = {"a": _tokens(61, vocab, 1), "b": _tokens(23, vocab, 2), "c": _tokens(3, vocab, 3), "d": _tokens(34, vocab, 4)}
    want = {k: _plain_logits(d, v) for k, v in reqs.items()}
    runner = _runner(d, dtype, page=8, pages=16, max_seqs=3)        # 128 tokens of cache for 121, three slots for four requests
    _poison(runner)
    s = TraceSession(runner)
    schedule = [[("a", 2), ("b", 17)], [("a", 30), ("c", 2), ("b", 1)], [("b", 1), ("c", 1)], [("a", 7), ("b", 2)],
                [("d", 9), ("a", 1), ("b", 2)], [("a", 1), ("d", 2)], [("d", 1), ("a", 19)], [("d", 22), ("a", 1)]]
    got = _replay(s, reqs, schedule)
    for k in reqs:
        assert got[k].shape[0] == len(reqs[k])
        assert _close(got[k], want[k], dtype), k
    assert runner.manager.num_free_slots() == 3 and runner.manager.check_invariants() == ""
    if dtype == "float32":
        # each alone, whole: what a row gives does not depend on the cut or the batch
        for k in reqs:
            alone = _replay(s, {k: reqs[k]}, [[(k, len(reqs[k]))]], first_step=100)[k]
            assert max_rel_diff(alone, got[k]) < 5e-6, k


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "T"])
def test_long_decoding_over_page_borders_and_windows(tmp_path, name, dtype):
    """150 tokens, all but six of them one by one: the windows (9, 16 and 37 keys) pass over decoded tokens
    many times and the window groups give their pages back on the way."""
    from vllm_oxide_b200.replay.trace import TraceSession
    d = _model_dir(tmp_path, name)
    toks = _tokens(150, _configs()[name].vocab, 9)
    want = _plain_logits(d, toks)
    runner = _runner(d, dtype, page=8, pages=20, max_seqs=2)
    _poison(runner)
    got = _replay(TraceSession(runner), {"a": toks}, [[("a", 6)]] + [[("a", 1)]] * 144)["a"]
    assert _close(got, want, dtype)


def test_a_window_one_token_off_would_show(tmp_path):
    """The plain model with every window one token longer differs from the engine by far more than the tolerance:
    the tests above can tell."""
    d = _model_dir(tmp_path, "A")
    from safetensors.torch import load_file
    cfg = json.load(open(os.path.join(d, "config.json")))
    toks = _tokens(60, 97, 1)
    tensors = load_file(os.path.join(d, "model.safetensors"))
    want = plain.forward(cfg, tensors, toks)
    for layer in cfg["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["left"]["mask"]["size"] += 1
    assert max_rel_diff(plain.forward(cfg, tensors, toks), want) > 1e-3


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_scheduler(tmp_path, graphs):
    """More requests than state slots and a pool that forces preemption and recomputation: every
    generated token is the plain model's argmax given what came before. With CUDA graphs the decode
    steps are recorded and replayed (nothing in these parts reads device data on the host)."""
    from vllm_oxide_b200.config import EngineConfig
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.sampling import SamplingParams
    d = _model_dir(tmp_path, "A")
    eng = EngineConfig(max_batch_tokens=64, max_seqs=3, max_model_len=64, block_size=8, num_pages=9, dtype="float32", cuda_graphs=graphs)
    llm = LLM(ModelRunner.from_dir(d, eng))
    prompts = [_tokens(n, 97, 20 + n) for n in (14, 9, 17, 5, 2)]
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=12, stop_token_ids=()))
    for prompt, o in zip(prompts, outs):
        assert len(o.token_ids) == 12
        logits = _plain_logits(d, list(prompt) + o.token_ids)
        for i, tok in enumerate(o.token_ids):
            row = logits[len(prompt) - 1 + i]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-3 * float(row.abs().max()):          # a near tie may fall either way
                assert tok == int(row.argmax()), (i, tok)
    assert llm.runner.manager.num_free_slots() == 3 and llm.runner.manager.check_invariants() == ""
    if graphs:
        assert llm.runner.decode_graphs and llm.runner._graphs


def test_greedy_generation_in_bfloat16_with_graphs(tmp_path):
    """bfloat16, sizes that take the tensor-core kernels, decode steps replayed from graphs: every generated token is
    the plain model's best, or as good as the best within what bfloat16 can tell apart."""
    from vllm_oxide_b200.config import EngineConfig
    from vllm_oxide_b200.engine import LLM, ModelRunner
    from vllm_oxide_b200.sampling import SamplingParams
    d = _model_dir(tmp_path, "T")
    prompts = [_tokens(n, 77, 40 + n) for n in (33, 6, 50)]
    eng = EngineConfig(max_batch_tokens=128, max_seqs=4, max_model_len=128, block_size=16, num_pages=24, dtype="bfloat16", cuda_graphs=True)
    llm = LLM(ModelRunner.from_dir(d, eng))
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=20, stop_token_ids=()))
    for prompt, o in zip(prompts, outs):
        assert len(o.token_ids) == 20
        logits = _plain_logits(d, list(prompt) + o.token_ids)
        for i, tok in enumerate(o.token_ids):
            row = logits[len(prompt) - 1 + i]
            assert float(row.max() - row[tok]) < 0.08 * float(row.abs().max()), (i, tok)
    assert llm.runner.decode_graphs and llm.runner._graphs


def test_command_line_generates_from_a_lomopel_folder(tmp_path):
    import subprocess
    import sys
    d = _model_dir(tmp_path, "B")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "vllm_oxide_b200", "generate", d, "--prompt-ids", "5,9,2,44", "--max-new", "6", "--dtype", "float32",
                        "--max-model-len", "64", "--max-batch-tokens", "64", "--max-seqs", "2", "--num-pages", "16"],
                       cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [int(x) for x in r.stdout.split()]
    toks = [5, 9, 2, 44]
    assert len(got) == 6
    logits = _plain_logits(d, toks + got)
    assert got[0] == int(logits[3].argmax())
