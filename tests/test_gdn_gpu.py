"""GPU parity of the Gated DeltaNet kernels (through the C ABI) with the oracle of the reference's token recurrence
(spinf_serve/models/qwen35/gdn.py:163-190), its tree driver (qwen.py:550-590) and the steps around it (qwen.py:640-673)."""

import numpy as np
import pytest
import torch

from oracle import gdn as OGD
from spinf_serve_b200 import packer as P
from spinf_serve_b200.gdn_plan import tree_plan

pytestmark = pytest.mark.gpu

Hk, Hv, D = 2, 4, 128


def _inputs(T, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn((T, Hk, D), generator=g), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn((T, Hk, D), generator=g), dim=-1).to(torch.bfloat16)
    v = torch.randn((T, Hv, D), generator=g).to(torch.bfloat16)
    gl = -torch.rand((T, Hv), generator=g) * 0.3  # log decay
    beta = torch.rand((T, Hv), generator=g).to(torch.bfloat16)
    return q, k, v, gl, beta


def _batch(seed, long_trunk=150):
    rng = np.random.default_rng(seed)
    pk = P.Packer(2048, 8192, align=True)
    for j in range(3):
        trunk = rng.integers(5, 50, int(rng.integers(20, long_trunk))).tolist()
        stems = [rng.integers(5, 50, 3).tolist() for _ in range(2)]
        prompts = []
        for i in range(int(rng.integers(2, 6))):
            prompts.append(trunk + stems[i % 2] + [60 + i] + rng.integers(5, 50, int(rng.integers(1, 9))).tolist())
        list(pk.push(j, P.build_grouped_tree(prompts, [P.ReadPlan.build([[5], [6, 7]]) for _ in prompts])))
    (b,) = list(pk.flush())
    return b


def test_tree_recurrence_vs_oracle(dev):
    """tries with nested forks: every branch starts from its parent's state; compared on every real row"""
    from spinf_serve_b200 import gdn

    for seed in (0, 1):
        b = _batch(seed)
        real = b.art >= 0
        q, k, v, gl, beta = _inputs(b.length, seed)
        plan_cpu = tree_plan(b.prev, real, "cpu", short=16)
        want = OGD.gdn_tree(q, k, v, gl, beta, plan_cpu, dtype=torch.float64)
        plan = tree_plan(b.prev, real, dev, short=16)
        got = gdn.gdn_tree(q.to(dev), k.to(dev), v.to(dev), gl.to(dev), beta.to(dev), plan).cpu()
        r = torch.from_numpy(real)
        err = (got[r].float() - want[r].float()).abs().max().item()
        print(f"seed {seed}: {plan.n_segments} segments, {len(plan.levels)} levels, max abs err {err:.3e} (|o| max {want[r].float().abs().max():.2f})")
        # segments longer than `short` run the chunked form, whose bf16 operands put it a few last bits from the fp64 recurrence
        assert err <= 2.0**-6 * want[r].float().abs().max().item()
        assert bool((got[~r] == 0).all())  # rows outside every segment are left zero


def test_recurrent_contract_states_and_gathered_rows(dev):
    """gathered form (idx None): final states written where ht_idx >= 0, children resume from them bit-exactly as one run"""
    from spinf_serve_b200 import gdn

    T = 90
    q, k, v, gl, beta = _inputs(T, 5)
    dq, dk, dv, dg, db = (t.to(dev) for t in (q, k, v, gl, beta))
    scale = D**-0.5
    cu_all = torch.tensor([0, T], dtype=torch.int64, device=dev)
    whole = gdn.recurrent(dq[None], dk[None], dv[None], dg[None], db[None], scale, cu_all, 1)[0]
    # the same sequence in two halves through a kept state
    st = torch.zeros((1, Hv, D, D), dtype=torch.float32, device=dev)
    first = gdn.recurrent(dq[None, :50], dk[None, :50], dv[None, :50], dg[None, :50], db[None, :50], scale,
                          torch.tensor([0, 50], dtype=torch.int64, device=dev), 1, ht=st, ht_idx=torch.zeros(1, dtype=torch.int64, device=dev))[0]
    second = gdn.recurrent(dq[None, 50:], dk[None, 50:], dv[None, 50:], dg[None, 50:], db[None, 50:], scale,
                           torch.tensor([0, 40], dtype=torch.int64, device=dev), 1, h0=st, h0_idx=torch.zeros(1, dtype=torch.int64, device=dev))[0]
    assert torch.equal(torch.cat([first, second]), whole)
    ref_state = torch.zeros((1, Hv, D, D), dtype=torch.float64)
    OGD.recurrent(q[:50], k[:50], v[:50], gl[:50], beta[:50], scale, [0, 50], ht=ref_state, ht_idx=[0], dtype=torch.float64)
    assert (st.cpu().double() - ref_state).abs().max().item() < 1e-4
    # a negative h0 index is the zero state; an empty segment touches nothing
    cu2 = torch.tensor([0, 0, 30], dtype=torch.int64, device=dev)
    out = gdn.recurrent(dq[None], dk[None], dv[None], dg[None], db[None], scale, cu2, 2, h0=st,
                        h0_idx=torch.tensor([0, -1], dtype=torch.int64, device=dev))[0]
    assert torch.equal(out[:30], whole[:30])


def test_prologue_and_epilogue_vs_oracle(dev):
    from spinf_serve_b200 import gdn

    b = _batch(3)
    real = b.art >= 0
    T = b.length
    plan = tree_plan(b.prev, real, "cpu")
    g = torch.Generator().manual_seed(9)
    conv_dim = 2 * Hk * D + Hv * D
    y = torch.randn((T, conv_dim + Hv * D + 2 * Hv), generator=g).to(torch.bfloat16)
    conv_w = (torch.randn((conv_dim, 4), generator=g) * 0.5).to(torch.bfloat16)
    A_log = torch.randn(Hv, generator=g) * 0.5
    dt_bias = torch.randn(Hv, generator=g)
    qo, ko, vo, zo, go, bo = OGD.prologue(y, plan.conv.numpy(), conv_w, A_log, dt_bias, Hk, D, Hv, D)
    q, k, v, z, gg, bb = gdn.prologue(y.to(dev), plan.conv.to(dev), conv_w.to(dev), A_log.to(dev), dt_bias.to(dev), Hk, D, Hv, D)
    for name, got, want in (("q", q, qo), ("k", k, ko), ("v", v, vo), ("beta", bb, bo)):
        diff = (got.cpu().float() - want.float()).abs()
        frac = (diff > 0).float().mean().item()
        print(f"prologue {name}: differing elements {frac:.4%}, max abs {diff.max():.3e}")
        assert frac < 5e-3 and diff.max() <= 2.0**-6 * want.float().abs().max()
    assert (gg.cpu() - go).abs().max() < 1e-5 * go.abs().max() + 1e-6
    assert torch.equal(z.cpu().reshape(T, Hv, D), zo)
    o = torch.randn((T, Hv, D), generator=g).to(torch.bfloat16)
    norm_w = (1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16)
    want = OGD.epilogue(o, zo, norm_w, 1e-6)
    got = gdn.epilogue(o.to(dev), z, norm_w.to(dev), 1e-6).cpu()
    diff = (got.float() - want.float()).abs()
    print(f"epilogue: differing elements {(diff > 0).float().mean():.4%}, max abs {diff.max():.3e}")
    assert (diff > 0).float().mean() < 5e-3 and diff.max() <= 2.0**-6 * want.float().abs().max()


def test_chunked_form_vs_its_oracle_and_the_token_recurrence(dev):
    """the chunked (WY) kernels against the oracle's restatement of the chunk pipeline (same rounding points: bf16 operands, fp32
    accumulation and state) and, more loosely, against the token recurrence they re-express; ragged segments (partial last chunks,
    a one-token segment), scattered stream rows, initial and final states by index"""
    from spinf_serve_b200 import gdn

    T = 700
    q, k, v, gl, beta = _inputs(T, 21)
    lens = [130, 64, 257, 1, 200]
    cu_cpu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    idx = torch.from_numpy(np.random.default_rng(3).permutation(T)[: cu_cpu[-1]].astype(np.int64))
    g0 = torch.Generator().manual_seed(5)
    h0 = torch.randn((2, Hv, D, D), generator=g0) * 0.05
    h0_idx = torch.tensor([1, -1, 0, 1, -1], dtype=torch.int64)
    ht_idx = torch.tensor([0, -1, 1, 2, -1], dtype=torch.int64)
    ht_ref, ht_ser = torch.zeros((3, Hv, D, D)), torch.zeros((3, Hv, D, D))
    want = OGD.chunked(q, k, v, gl, beta, D**-0.5, cu_cpu, idx.numpy(), h0, h0_idx.numpy(), ht_ref, ht_idx.numpy())
    serial = OGD.recurrent(q, k, v, gl, beta, D**-0.5, cu_cpu, idx.numpy(), h0, h0_idx.numpy(), ht_ser, ht_idx.numpy())
    ht = torch.zeros((3, Hv, D, D), device=dev)
    got = gdn.chunked(q.to(dev), k.to(dev), v.to(dev), gl.to(dev), beta.to(dev), D**-0.5, torch.from_numpy(cu_cpu).to(dev), cu_cpu,
                      h0=h0.to(dev), h0_idx=h0_idx.to(dev), ht=ht, ht_idx=ht_idx.to(dev), idx=idx.to(dev))[0].cpu()
    touched = torch.zeros(T, dtype=torch.bool)
    touched[idx] = True
    scale_o, scale_s = want.float().abs().max().item(), ht_ref.abs().max().item()
    e_o = (got.float() - want.float())[touched].abs().max().item()
    e_s = (ht.cpu() - ht_ref).abs().max().item()
    e_ser = (got.float() - serial.float())[touched].abs().max().item()
    print(f"chunked GDN: output err {e_o:.3e} of {scale_o:.3f} (vs token recurrence {e_ser:.3e}), state err {e_s:.3e} of {scale_s:.3f}")
    assert e_o <= 2.0**-6 * scale_o and e_s <= 2e-3 * scale_s   # same roundings: a few bf16 last-bit flips apart
    assert e_ser <= 2e-2 * scale_o                              # the two forms differ by the chunk pipeline's bf16 operands
    assert bool((got[~touched] == 0).all())


@pytest.mark.parametrize("scan", ["mma", "tc"])
def test_fused_tree_kernels_vs_oracles(dev, scan):
    """the one-launch-per-level kernels (every segment in the chunked form, light siblings packed into shared tiles, a parent's
    state read once per group) on tries with nested forks: against the chunk-form oracle (same rounding points) and the fp64
    token recurrence; rows outside every segment stay zero; the per-call kernels agree to the chunk pipeline's roundings"""
    from spinf_serve_b200 import gdn

    old, gdn.SCAN = gdn.SCAN, scan
    try:
        _fused_cases(dev, gdn, scan)
    finally:
        gdn.SCAN = old


def _fused_cases(dev, gdn, scan):
    for seed, long_trunk in ((0, 150), (1, 150), (2, 700)):
        b = _batch(seed, long_trunk)
        real = b.art >= 0
        q, k, v, gl, beta = _inputs(b.length, seed)
        plan_cpu = tree_plan(b.prev, real, "cpu")
        want64 = OGD.gdn_tree(q, k, v, gl, beta, plan_cpu, dtype=torch.float64)
        want_c = OGD.gdn_tree(q, k, v, gl, beta, plan_cpu, form="chunked")
        plan = tree_plan(b.prev, real, dev)
        assert plan.fused is not None and plan.fused.plan_tokens == int(real.sum())
        dq, dk, dv, dg, db = (t.to(dev) for t in (q, k, v, gl, beta))
        got = gdn.gdn_tree(dq, dk, dv, dg, db, plan).cpu()
        gdn.FUSED = False
        try:
            calls = gdn.gdn_tree(dq, dk, dv, dg, db, plan).cpu()
        finally:
            gdn.FUSED = True
        r = torch.from_numpy(real)
        big = want64[r].float().abs().max().item()
        e64 = (got[r].float() - want64[r].float()).abs().max().item()
        ec = (got[r].float() - want_c[r].float()).abs().max().item()
        ek = (got[r].float() - calls[r].float()).abs().max().item()
        units = [int(lv[2].shape[0]) for lv in plan.fused.levels]
        print(f"scan {scan}, seed {seed}: {plan.n_segments} segments, units per level {units}: vs fp64 recurrence {e64:.3e}, vs chunk-form oracle {ec:.3e}, "
              f"vs per-call kernels {ek:.3e} (|o| max {big:.3f})")
        assert ec <= 2.0**-6 * big and e64 <= 2e-2 * big and ek <= 2e-2 * big
        assert bool((got[~r] == 0).all())


@pytest.mark.parametrize("scan", ["mma", "tc"])
def test_fused_tree_rows_do_not_depend_on_the_packing(dev, scan):
    """a content's recurrent outputs are bit-identical whether its trie runs alone or packed after others (light siblings share
    tiles, groups share launches: none of it may reach the values)"""
    from spinf_serve_b200 import gdn

    rng = np.random.default_rng(11)
    trees = []
    for j in range(3):
        trunk = rng.integers(5, 50, int(rng.integers(70, 300))).tolist()
        prompts = [trunk + [60 + i] + rng.integers(5, 50, int(rng.integers(3, 30))).tolist() for i in range(int(rng.integers(3, 9)))]
        trees.append(P.build_grouped_tree(prompts, [P.ReadPlan.build([[5], [6, 7]]) for _ in prompts]))

    def run(order):
        pk = P.Packer(4096, 8192, align=True)
        for j in order:
            list(pk.push(j, trees[j]))
        (b,) = list(pk.flush())
        g = torch.Generator().manual_seed(3)
        # every job draws its own inputs from its own generator, so that a job's tokens are the same in both packings
        q = torch.zeros((b.length, Hk, D), dtype=torch.bfloat16)
        k, v = torch.zeros_like(q), torch.zeros((b.length, Hv, D), dtype=torch.bfloat16)
        gl, beta = torch.zeros((b.length, Hv)), torch.zeros((b.length, Hv), dtype=torch.bfloat16)
        where = {}
        for o in b.owners:
            gj = torch.Generator().manual_seed(100 + o.job_id)
            n = o.n_tokens
            sl = slice(o.start, o.start + n)
            q[sl] = torch.nn.functional.normalize(torch.randn((n, Hk, D), generator=gj), dim=-1).to(torch.bfloat16)
            k[sl] = torch.nn.functional.normalize(torch.randn((n, Hk, D), generator=gj), dim=-1).to(torch.bfloat16)
            v[sl] = torch.randn((n, Hv, D), generator=gj).to(torch.bfloat16)
            gl[sl] = -torch.rand((n, Hv), generator=gj) * 0.3
            beta[sl] = torch.rand((n, Hv), generator=gj).to(torch.bfloat16)
            where[o.job_id] = sl
        plan = tree_plan(b.prev, b.art >= 0, dev)
        out = gdn.gdn_tree(q.to(dev), k.to(dev), v.to(dev), gl.to(dev), beta.to(dev), plan).cpu()
        return {j: out[sl] for j, sl in where.items()}

    old, gdn.SCAN = gdn.SCAN, scan
    try:
        alone = run([1])
        packed = run([0, 2, 1])
    finally:
        gdn.SCAN = old
    assert torch.equal(alone[1], packed[1])
