"""The Rotepel decoder in the engine against the plain implementation (tests/plain/rotepel_plain.py):
small configurations made here, random weights, float32 and bfloat16. Each mechanism alone (a model
of one layer, and the kernels on inputs made so that a fault shows), whole prompts against tokens
one by one, portions down to two tokens, unequal requests side by side against each alone, pages
and state slots that are given back and used again, and greedy generation through `LLM`."""
import json
import os
import random

import pytest
import torch

from tests.plain import rotepel_plain as plain
from tests.util import max_rel_diff

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _layer(kind, **kw):
    from vllm_oxide_b200.config import RotepelLayer
    return RotepelLayer(type=kind, **kw)


def _configs():
    from vllm_oxide_b200.config import RotepelConfig
    delta = _layer("general_delta", heads=2, dim=16, decay_rank=4, ff=96)
    delta_wide = _layer("general_delta", heads=1, dim=40, decay_rank=6, ff=0)
    ret = _layer("retention", heads=3, dim=32, vdim=16, decay=(0.9, 0.97, 0.995), rot_dims=16, rot_base=10000.0, ff=80)
    ret_one = _layer("retention", heads=1, dim=16, vdim=48, decay=(0.99,), rot_dims=16, rot_base=500.0, ff=72)
    lat = _layer("latent_attention", heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.3, rot_dims=8, rot_base=10000.0, ff=0)
    lat_one = _layer("latent_attention", heads=1, dim=32, rot_dim=16, vdim=8, kv_rank=24, scale=0.2, rot_dims=16, rot_base=300.0, ff=112)
    # latent and rotated sizes that are multiples of 16: in bfloat16 prompt portions take the tensor-core kernel
    lat_16 = _layer("latent_attention", heads=5, dim=16, rot_dim=16, vdim=8, kv_rank=48, scale=0.25, rot_dims=16, rot_base=1000.0, ff=64)
    return {
        # three streams, one norm group, a loop of three passes over the first two layers
        "A": RotepelConfig(vocab=97, width=64, layers=(delta, lat, ret), norm_eps=1e-5, norm_groups=1, streams=3, loop=(0, 2, 3)),
        # no streams at all (the plain residual), three norm groups, single heads, no loop
        "B": RotepelConfig(vocab=131, width=96, layers=(ret_one, delta_wide, lat_one), norm_eps=1e-6, norm_groups=3, streams=None),
        # one stream with coefficients of its own, four groups, a loop that runs once, attention twice
        "C": RotepelConfig(vocab=64, width=64, layers=(lat, delta, lat_one), norm_eps=1e-5, norm_groups=4, streams=1, loop=(1, 3, 1)),
        # attention whose sizes the tensor-core kernel takes, twice in a loop, beside retention; 42 is no multiple of 4
        "T": RotepelConfig(vocab=77, width=42, layers=(lat_16, ret_one), norm_eps=1e-5, norm_groups=3, streams=2, loop=(0, 1, 2)),
        "delta": RotepelConfig(vocab=50, width=48, layers=(delta,), norm_eps=1e-5, norm_groups=2, streams=2),
        "retention": RotepelConfig(vocab=50, width=48, layers=(ret,), norm_eps=1e-5, norm_groups=2, streams=2),
        "latent": RotepelConfig(vocab=50, width=48, layers=(lat,), norm_eps=1e-5, norm_groups=2, streams=2),
    }


def _model_dir(tmp_path, name, seed=11):
    from vllm_oxide_b200.weights import write_random_model
    d = os.path.join(str(tmp_path), f"rotepel_{name}_{seed}")
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


# float32: the engine against float64, rounding over a few hundred operations per logit. bfloat16: every projection's
# input and output, the cache and the gated outputs are rounded to 8 mantissa bits (2^-9 relative each), some fifteen
# roundings a layer run over up to seven layer runs: 2^-9 * sqrt(100) ~ 2e-2 of the largest logit as a typical row,
# three times that for the worst logit of all rows.
TOL = {"float32": 3e-5, "bfloat16": 6e-2}


def _close(got, want, dtype) -> bool:
    """float32: every logit within TOL of the largest. bfloat16: the typical row tight (root mean square of a row's
    error against that of its logits, averaged over the rows, below 2.5e-2: measured 0.6e-2 to 1.8e-2 on these models,
    the same with either attention kernel) and no logit anywhere off by more than a tenth of the largest. A key that
    is skipped, a wrong page or a lost state moves rows by far more than either bound."""
    if dtype == "float32":
        return max_rel_diff(got, want) < TOL[dtype]
    err = (got.double() - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()
    return float(err.mean()) < 2.5e-2 and max_rel_diff(got, want) < 0.1


def _poison(runner):
    """Whatever lies in pages and slots that nobody holds must never be read."""
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


# ------------------------------------------------------------------------------------ kernels alone
def test_stream_norm_kernel_pending_write_groups_and_row_list():
    from vllm_oxide_b200 import kernels
    torch.manual_seed(0)
    for S, W, groups, T in ((1, 64, 1, 5), (3, 96, 4, 7), (8, 40, 5, 3), (2, 42, 3, 4)):       # the last: no 16-byte accesses
        x = torch.randn(T, S, W, device=DEV)
        y = torch.randn(T, W, device=DEV)
        mix, outc, inc, w = torch.randn(S, S, device=DEV), torch.randn(S, device=DEV), torch.randn(S, device=DEV), torch.randn(W, device=DEV)
        new = torch.einsum("st,rsw->rtw", mix.double(), x.double()) + outc.double()[None, :, None] * y.double()[:, None, :]
        want = plain.group_rms_norm(torch.einsum("t,rtw->rw", inc.double(), new), w.double(), 1e-5, groups)
        # only looked at: a row list leaves the streams alone
        rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
        out = torch.empty(2, W, device=DEV)
        before = x.clone()
        kernels.stream_norm(x, y, mix.contiguous(), outc, inc, w, groups, 1e-5, out, rows)
        assert torch.equal(x, before)
        assert max_rel_diff(out, want[[T - 1, 0]]) < 1e-5
        # stored, and the result written twice side by side
        out2 = torch.empty(T, 2, W, device=DEV)
        kernels.stream_norm(x, y, mix.contiguous(), outc, inc, w, groups, 1e-5, out2)
        assert max_rel_diff(x, new) < 1e-5
        assert max_rel_diff(out2[:, 0], want) < 1e-5 and torch.equal(out2[:, 0], out2[:, 1])
        # no pending write, no read coefficients: the norm of the plain sum
        out3 = torch.empty(T, W, device=DEV)
        kernels.stream_norm(x, None, None, None, None, w, groups, 1e-5, out3)
        assert max_rel_diff(out3, plain.group_rms_norm(x.double().sum(1), w.double(), 1e-5, groups)) < 1e-5


def _scan_reference(mode, r, k, v, w, b, u, S0):
    """One request, one head, float64: returns (o [T, V], final state)."""
    S = S0.clone()
    o = []
    for t in range(r.shape[0]):
        if mode == 0:
            S = w[t][:, None] * S - b[t][:, None] * (u[t] @ S)[None, :] + k[t][:, None] * v[t][None, :]
        else:
            S = w * S + k[t][:, None] * v[t][None, :]
        o.append(S.T @ r[t])
    return torch.stack(o), S


@pytest.mark.parametrize("mode,K,V", [(0, 16, 16), (0, 40, 40), (0, 136, 24), (1, 32, 16), (1, 16, 48), (1, 300, 8), (0, 264, 8)])
def test_recurrence_scan_kernel_sizes_portions_and_slots(mode, K, V):
    """Two requests with unequal portions in one launch, in slots 2 and 0 of a state tensor whose other
    slots must stay as they are; then the rest of both, token by token for one of them. The outputs
    equal the float64 recurrence, and cutting a request differently gives the same bits."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(1)
    H, lens = 2, (37, 9)
    T = sum(lens)

    def data():
        d = dict(r=torch.randn(T, H * K, device=DEV), k=torch.randn(T, H * K, device=DEV) * 0.3, v=torch.randn(T, H * V, device=DEV))
        if mode == 0:
            d["w"] = torch.rand(T, H * K, device=DEV) * 0.4 + 0.58
            u = torch.nn.functional.normalize(d["k"].view(T, H, K), dim=-1).reshape(T, H * K).contiguous()
            d["u"], d["b"] = u, (torch.rand(T, H * K, device=DEV) * u).contiguous()
        else:
            d["w"], d["b"], d["u"] = torch.tensor([0.95, 0.999], device=DEV), None, None
        return d
    d = data()
    starts = [0, lens[0], T]

    def run(cuts):
        """cuts: per request the portion sizes; every launch takes the next portion of each request that has one."""
        state = torch.full((4, H, K, V), 7.0, device=DEV)
        state[2].zero_()
        state[0].zero_()
        out = torch.zeros(T, H * V, device=DEV)
        done = [0, 0]
        slots = torch.tensor([2, 0], dtype=torch.int32, device=DEV)
        for step in range(max(len(c) for c in cuts)):
            rows, ss = [], [0]
            for s in range(2):
                n = cuts[s][step] if step < len(cuts[s]) else 0
                rows += list(range(starts[s] + done[s], starts[s] + done[s] + n))
                done[s] += n
                ss.append(len(rows))
            idx = torch.tensor(rows, device=DEV)
            o = torch.empty(len(rows), H * V, device=DEV)
            sel = {n: (t[idx].contiguous() if t is not None and t.dim() == 2 else t) for n, t in d.items()}
            kernels.recurrence_scan(mode, sel["r"], sel["k"], sel["v"], sel["w"], sel["b"], sel["u"], state,
                                    torch.tensor(ss, dtype=torch.int32, device=DEV), slots, 2, H, o)
            out[idx] = o
        assert done == list(lens)
        return out, state
    whole, st = run([[37], [9]])
    assert torch.all(st[1] == 7.0) and torch.all(st[3] == 7.0)
    cut, st2 = run([[2, 16, 1, 17, 1], [1] * 9])
    assert torch.equal(whole, cut) and torch.equal(st, st2)
    for s, slot in ((0, 2), (1, 0)):
        for h in range(H):
            sl = slice(starts[s], starts[s + 1])
            rk = lambda t, n: t[sl, h * n:(h + 1) * n].double().cpu()
            w = rk(d["w"], K) if mode == 0 else d["w"][h].double().cpu()
            o_ref, S_ref = _scan_reference(mode, rk(d["r"], K), rk(d["k"], K), rk(d["v"], V), w,
                                           rk(d["b"], K) if mode == 0 else None, rk(d["u"], K) if mode == 0 else None,
                                           torch.zeros(K, V, dtype=torch.float64))
            assert max_rel_diff(whole[sl, h * V:(h + 1) * V].cpu(), o_ref) < 2e-5
            assert max_rel_diff(st[slot, h].cpu(), S_ref) < 2e-5


def test_retention_remembers_a_token_far_back():
    """A decay close to one: the first token's key and value, made large, still set the output 300
    tokens later (a state that was lost or zeroed on the way would give something else)."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(2)
    T, K, V = 301, 16, 16
    q, k, v = torch.randn(T, K, device=DEV) * 0.1, torch.randn(T, K, device=DEV) * 0.1, torch.randn(T, V, device=DEV) * 0.1
    k[0], v[0], q[T - 1] = 0.0, 0.0, 0.0
    k[0, 3], v[0, 5], q[T - 1, 3] = 10.0, 10.0, 1.0
    state = torch.zeros(1, 1, K, V, device=DEV)
    o = torch.empty(T, V, device=DEV)
    slots = torch.zeros(1, dtype=torch.int32, device=DEV)
    decay = torch.tensor([0.999], device=DEV)
    for lo, hi in ((0, 120), (120, 122), (122, 300), (300, 301)):
        kernels.recurrence_scan(1, q[lo:hi], k[lo:hi], v[lo:hi], decay, None, None, state,
                                torch.tensor([0, hi - lo], dtype=torch.int32, device=DEV), slots, 1, 1, o[lo:hi])
    o_ref, _ = _scan_reference(1, q.double().cpu(), k.double().cpu(), v.double().cpu(), torch.tensor(0.999, dtype=torch.float64), None, None,
                               torch.zeros(K, V, dtype=torch.float64))
    assert abs(float(o_ref[-1, 5]) - 100 * 0.999 ** 300) < 1.0          # the far token is what the last output is made of
    assert max_rel_diff(o.cpu(), o_ref) < 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attend_kernel_far_key_page_borders_and_first_tokens(dtype):
    """Keys in pages that are scattered over the pool; for chosen rows one key (the very first, the
    last of a page, the first of the next page, the row's own, one far back among hundreds) is made to
    dominate the softmax, so that a key that is skipped, or read from the wrong slot, changes the row."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(3)
    H, L, R, page, n = 3, 40, 8, 8, 419
    pages = -(-n // page)
    perm = torch.randperm(pages + 5)[:pages]
    c = (torch.randn(n, L) * 0.5)
    kr = torch.randn(n, R) * 0.5
    q_lat, q_rot = torch.randn(n, H, L) * 0.3, torch.randn(n, H, R) * 0.3
    scale = 0.37
    # (row, key): the key that row must find
    marked = [(n - 1, 0), (n - 1 - page, 7), (300, 8), (200, 200), (n - 2, 23), (5, 0), (0, 0), (64, 63), (65, 64)]
    for row, key in marked:
        c[key] = torch.randn(L) * 0.5
    for row, key in marked:
        q_lat[row, :, :] = 6.0 * c[key] / c[key].norm() ** 2 / scale * 3.0
    lat_c = torch.full((pages + 5, 1, page, L), float("nan"), dtype=dtype, device=DEV)
    kr_c = torch.full((pages + 5, 1, page, R), float("nan"), dtype=dtype, device=DEV)
    slot = perm[torch.arange(n) // page] * page + torch.arange(n) % page
    lat_c.view(-1, L)[slot.to(DEV)] = c.to(device=DEV, dtype=dtype)
    kr_c.view(-1, R)[slot.to(DEV)] = kr.to(device=DEV, dtype=dtype)
    table = torch.full((2, pages + 3), -1, dtype=torch.int32, device=DEV)
    table[1, :pages] = perm.to(torch.int32)
    rows = torch.arange(n)
    out = torch.empty(n, H, L, dtype=dtype, device=DEV)
    kernels.latent_attend(q_lat.to(DEV), q_rot.to(DEV), lat_c, kr_c, table, torch.ones(n, dtype=torch.int32, device=DEV),
                          rows.to(device=DEV, dtype=torch.int32), scale, out)
    cc, kk = c.to(dtype).double(), kr.to(dtype).double()
    score = (torch.einsum("ihl,jl->hij", q_lat.double(), cc) + torch.einsum("ihr,jr->hij", q_rot.double(), kk)) * scale
    score = score.masked_fill(~torch.ones(n, n, dtype=torch.bool).tril(), float("-inf"))
    p = torch.softmax(score, -1)
    want = torch.einsum("hij,jl->ihl", p, cc)
    for row, key in marked:
        assert float(p[:, row, key].min()) > 0.5, (row, key)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert max_rel_diff(out.cpu(), want) < tol
    for row, key in marked:
        assert max_rel_diff(out[row].cpu(), want[row]) < tol, (row, key)
    # a padding row (position -1) attends to nothing and reads no table
    pos = rows.clone()
    pos[7] = -1
    out2 = torch.empty_like(out)
    kernels.latent_attend(q_lat.to(DEV), q_rot.to(DEV), lat_c, kr_c, table, torch.ones(n, dtype=torch.int32, device=DEV),
                          pos.to(device=DEV, dtype=torch.int32), scale, out2)
    assert torch.all(out2[7] == 0) and torch.equal(out2[8:], out[8:])


@pytest.mark.parametrize("H,L,R", [(5, 48, 16), (9, 128, 32), (3, 288, 32), (2, 512, 64)])
def test_latent_attend_tensor_core_kernel_against_float64(H, L, R):
    """Prompt portions on the tensor cores: two requests in one launch, the second with 37 keys already cached,
    pages scattered, head counts that leave a block partly empty, tiles of 16 tokens that end inside a portion,
    one dominant key far back and one at the row's own position; latents of one warp per head (up to 256
    columns) and of two (288, 512), key tiles that fit the registers fetched ahead and ones that do not."""
    from vllm_oxide_b200 import kernels
    torch.manual_seed(4)
    page, scale = 8, 0.4
    lens, ctxs = (100, 50), (0, 37)
    total = [c + n for c, n in zip(ctxs, lens)]
    pages_per = [-(-t // page) for t in total]
    perm = torch.randperm(sum(pages_per) + 4)
    tables = torch.full((2, max(pages_per) + 2), -1, dtype=torch.int32)
    tables[0, :pages_per[0]] = perm[:pages_per[0]].to(torch.int32)
    tables[1, :pages_per[1]] = perm[pages_per[0]:sum(pages_per)].to(torch.int32)
    lat_c = torch.full((sum(pages_per) + 4, 1, page, L), float("nan"), dtype=torch.bfloat16, device=DEV)
    kr_c = torch.full((sum(pages_per) + 4, 1, page, R), float("nan"), dtype=torch.bfloat16, device=DEV)
    c = [torch.randn(t, L) * 0.5 for t in total]
    kr = [torch.randn(t, R) * 0.5 for t in total]
    T = sum(lens)
    q_lat, q_rot = torch.randn(T, H, L) * 0.3, torch.randn(T, H, R) * 0.3
    q_lat[99] = 8.0 * c[0][3] / c[0][3].norm() ** 2 / scale            # row 99 of request 0 looks for key 3
    q_lat[100 + 20] = 8.0 * c[1][57] / c[1][57].norm() ** 2 / scale    # row 20 of request 1 (position 57) looks for its own key
    for s in range(2):
        idx = torch.arange(total[s])
        slot = tables[s, idx // page].long() * page + idx % page
        lat_c.view(-1, L)[slot.to(DEV)] = c[s].to(device=DEV, dtype=torch.bfloat16)
        kr_c.view(-1, R)[slot.to(DEV)] = kr[s].to(device=DEV, dtype=torch.bfloat16)
    positions = torch.cat([torch.arange(ctxs[s], total[s]) for s in range(2)]).to(device=DEV, dtype=torch.int32)
    starts = torch.tensor([0, lens[0], T], dtype=torch.int32, device=DEV)
    out = torch.empty(T, H, L, dtype=torch.bfloat16, device=DEV)
    assert kernels.latent_attend_tc_supported(H, L, R) and not kernels.latent_attend_tc_supported(H, 40, 8)
    kernels.latent_attend_tc(q_lat.to(DEV), q_rot.to(DEV), lat_c, kr_c, tables.to(DEV), starts, positions, 2, 100, scale, out)
    r0 = 0
    for s in range(2):
        cc, kk = c[s].bfloat16().double(), kr[s].bfloat16().double()
        ql, qr = q_lat[r0:r0 + lens[s]].bfloat16().double(), q_rot[r0:r0 + lens[s]].bfloat16().double()
        score = (torch.einsum("ihl,jl->hij", ql, cc) + torch.einsum("ihr,jr->hij", qr, kk)) * scale
        visible = torch.arange(total[s])[None, :] <= torch.arange(ctxs[s], total[s])[:, None]
        p = torch.softmax(score.masked_fill(~visible, float("-inf")), -1)
        want = torch.einsum("hij,jl->ihl", p, cc)
        assert max_rel_diff(out[r0:r0 + lens[s]].cpu(), want) < 1.5e-2, s
        if s == 0:
            assert float(p[:, 99, 3].min()) > 0.5            # the far key is what row 99 is made of
        else:
            assert float(p[:, 20, 57].min()) > 0.5
        r0 += lens[s]


# ------------------------------------------------------------------------------------ models in the engine
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["delta", "retention", "latent"])
def test_each_mixer_alone_whole_prompt_and_token_by_token(tmp_path, name, dtype):
    from vllm_oxide_b200.replay.trace import TraceSession
    d = _model_dir(tmp_path, name)
    toks = _tokens(45, 50, 5)
    want = _plain_logits(d, toks)
    runner = _runner(d, dtype)
    _poison(runner)
    s = TraceSession(runner)
    whole = _replay(s, {"a": toks}, [[("a", 45)]])["a"]
    assert max_rel_diff(whole, want) < TOL[dtype]
    # most of it at once, the rest one by one, in the slot and the pages that were just given back
    _poison(runner)
    single = _replay(s, {"b": toks}, [[("b", 19)]] + [[("b", 1)]] * 26, first_step=10)["b"]
    assert max_rel_diff(single, want) < TOL[dtype]
    if dtype == "float32":
        assert max_rel_diff(single, whole) < 3e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "T"])
def test_portions_unequal_batches_and_reuse(tmp_path, name, dtype):
    """Three requests of unequal length in a pool that cannot hold them all at once: portions from 2
    tokens up beside single tokens, a request that sits out a step, a fourth request that takes over a
    slot and pages that were given back in the middle. Every row equals the plain model's."""
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
def test_long_decoding_over_page_borders(tmp_path, dtype):
    from vllm_oxide_b200.replay.trace import TraceSession
    d = _model_dir(tmp_path, "A")
    toks = _tokens(150, 97, 9)
    want = _plain_logits(d, toks)
    runner = _runner(d, dtype, page=8, pages=20, max_seqs=2)
    _poison(runner)
    got = _replay(TraceSession(runner), {"a": toks}, [[("a", 6)]] + [[("a", 1)]] * 144)["a"]
    assert max_rel_diff(got, want) < TOL[dtype]


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
        seq = list(prompt)
        logits = _plain_logits(d, seq + o.token_ids)
        for i, tok in enumerate(o.token_ids):
            row = logits[len(prompt) - 1 + i]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-3 * float(row.abs().max()):          # a near tie may fall either way
                assert tok == int(row.argmax()), (i, tok)
    assert llm.runner.manager.num_free_slots() == 3 and llm.runner.manager.check_invariants() == ""
    if graphs:
        assert llm.runner.decode_graphs and llm.runner._graphs


def test_command_line_generates_from_a_rotepel_folder(tmp_path):
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
