"""CPU unit tests of the framework's pure logic: schedule, partitioning, optimizers, configs, data,
load-balance losses, MoE index math, native signature table."""
import glob
import math
import re
from dataclasses import dataclass
from datetime import timedelta
from functools import partial
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


# ------------------------------------------------------------------------------------------------ schedule
@pytest.mark.parametrize("P", [1, 2, 3, 4, 8])
def test_schedule_simulation(P):
    from pithtrain_b200.dualpipe.schedule import build_schedule, simulate

    for N in (2 * P, 2 * P + 1, 3 * P + 2, 4 * P):
        simulate(P, N)
        for r in range(P):
            acts = build_schedule(P, r, N)
            f = sum(a.kind in ("F", "FB") for a in acts)
            assert f == 2 * N  # every micro-batch passes both local chunks
    with pytest.raises(AssertionError):
        build_schedule(P, 0, 2 * P - 1)


def test_layer_partition_properties():
    from pithtrain_b200.dualpipe.dualpipev import layer_partition

    for L in range(1, 70):
        for S in (1, 2, 4, 6, 8, 16):
            parts = [layer_partition(L, S, i) for i in range(S)]
            flat = [x for p in parts for x in p]
            assert flat == list(range(L))
            sizes = [len(p) for p in parts]
            assert max(sizes) - min(sizes) <= 1
            if S > 2 and L % S and L % S <= S - 2:
                assert sizes[0] == min(sizes) and sizes[-1] == min(sizes)  # edges stay light
    assert [len(layer_partition(27, 4, i)) for i in range(4)] == [7, 7, 7, 6]


# ------------------------------------------------------------------------------------------------ config
def test_slotted_default_and_json():
    from pithtrain_b200.config import SlottedDefault

    @dataclass(init=False, slots=True)
    class Cfg(SlottedDefault):
        need: int
        opt: int = 3
        path: Path = Path("/x")
        t: timedelta = timedelta(minutes=1)
        fn: object = None

    c = Cfg()
    assert c.opt == 3 and not hasattr(c, "need")
    c.fn = partial(math.pow, y=2)
    j = c.to_json_dict()
    assert j["path"] == "/x" and j["t"] == 60.0 and j["fn"] == "pow(y=2)" and "need" not in j


def test_wsd_schedule():
    from pithtrain_b200.modules.training import wsd_lambda

    fn = wsd_lambda(100, 1.0, start_lr=0.0, warmup_ratio=0.1, final_lr=0.1, decay_ratio=0.2, decay_shape="linear")
    assert fn(0) == 0.0 and abs(fn(5) - 0.5) < 1e-9 and fn(10) == 1.0 and fn(79) == 1.0
    assert abs(fn(90) - 0.55) < 1e-9 and abs(fn(100) - 0.1) < 1e-9
    cos = wsd_lambda(100, 1.0, decay_ratio=0.5, decay_shape="cosine")
    assert abs(cos(75) - 0.5) < 1e-9
    with pytest.raises(ValueError):
        wsd_lambda(10, 1.0, warmup_ratio=0.6, decay_ratio=0.6)


# ------------------------------------------------------------------------------------------------ optimizers
def test_is_muon_param_table():
    from pithtrain_b200.modules.training import is_muon_param

    m2, m3, m1 = torch.zeros(4, 4), torch.zeros(2, 4, 4), torch.zeros(4)
    yes = ["layers.0.self_attn.q_proj.weight", "layers.0.self_attn.kv_b_proj.weight", "layers.1.mlp.gate_proj.weight",
           "layers.1.mlp.shared_experts.down_proj.weight"]
    for n in yes:
        assert is_muon_param(n, m2), n
    assert is_muon_param("layers.1.mlp.experts.gate_proj.weight", m3)
    assert is_muon_param("layers.1.mlp.experts.gate_up_proj", m3)
    no = [("layers.0.input_layernorm.weight", m1), ("layers.0.self_attn.q_proj.bias", m1),
          ("layers.0.mlp.experts.gate_up_proj_bias", m2), ("embed_tokens.weight", m2), ("lm_head.weight", m2),
          ("layers.0.mlp.gate.weight", m2), ("layers.0.mlp.router.weight", m2), ("layers.0.self_attn.sinks", m1)]
    for n, t in no:
        assert not is_muon_param(n, t), n


@pytest.mark.parametrize("shape", [(16, 64), (64, 16), (3, 24, 40)])
def test_newton_schulz_orthogonalises(shape):
    from pithtrain_b200.modules.optimizer import muon_scale_factor, zeropower_via_newtonschulz5

    torch.manual_seed(0)
    G = torch.randn(*shape)
    X = zeropower_via_newtonschulz5(G, steps=5).float()
    sv = torch.linalg.svdvals(X)
    assert float(sv.min()) > 0.5 and float(sv.max()) < 1.5
    U, _, Vh = torch.linalg.svd(G, full_matrices=False)
    cos = (X * (U @ Vh)).sum() / (X.norm() * (U @ Vh).norm())
    assert float(cos) > 0.97
    assert muon_scale_factor(16, 64) == 0.2 * 8.0


def test_muon_step_matches_formula():
    from pithtrain_b200.modules.optimizer import Muon, muon_scale_factor, zeropower_via_newtonschulz5

    torch.manual_seed(1)
    p = torch.nn.Parameter(torch.randn(8, 12))
    g1, g2 = torch.randn(8, 12), torch.randn(8, 12)
    opt = Muon([p], lr=0.1, momentum=0.9, weight_decay=0.05)
    w, buf = p.detach().clone(), torch.zeros(8, 12)
    for g in (g1, g2):
        p.grad = g.clone()
        opt.step()
        buf = buf.lerp(g, 0.1)
        upd = g.lerp(buf, 0.9)
        o = zeropower_via_newtonschulz5(upd).float() * muon_scale_factor(8, 12)
        w = w * (1 - 0.1 * 0.05) - 0.1 * o
    assert torch.allclose(p.detach(), w, atol=1e-5)
    p.grad = g1.bfloat16().float()
    opt.step()  # bf16-rounded gradients are fine


def test_adamw_matches_torch():
    from pithtrain_b200.modules.optimizer import AdamW

    torch.manual_seed(2)
    a = torch.nn.Parameter(torch.randn(5, 7))
    b = torch.nn.Parameter(a.detach().clone())
    mine, ref = AdamW([a], lr=1e-2, weight_decay=0.1), torch.optim.AdamW([b], lr=1e-2, weight_decay=0.1)
    for _ in range(3):
        g = torch.randn(5, 7)
        a.grad, b.grad = g.clone(), g.clone()
        mine.step(); ref.step()
    assert torch.allclose(a, b, atol=1e-6)


# ------------------------------------------------------------------------------------------------ load balance
def test_load_balance_losses():
    from pithtrain_b200.modules.load_balance import (MoELoadBalanceLossInjector, SequenceLevelLoadBalanceLoss,
                                                     force_balance, make_load_balance_loss_fn)

    torch.manual_seed(0)
    n, E, k = 64, 8, 2
    scores = torch.rand(n, E).softmax(-1).requires_grad_()
    idx = torch.topk(scores, k).indices
    fn = make_load_balance_loss_fn("micro-batch", 0.5)
    f = torch.bincount(idx.flatten(), minlength=E).float() / (n * k)
    assert torch.allclose(fn(scores, idx, E, k), 0.5 * E * (f * scores.mean(0)).sum())
    bal = force_balance(E)(idx)
    assert torch.bincount(bal.flatten(), minlength=E).tolist() == [n * k // E] * E
    g = make_load_balance_loss_fn("global-batch", 1.0)
    l1 = g(scores, bal, E, k)
    assert abs(float(l1) - 1.0) < 1e-5  # perfectly balanced counts: E * sum(1/E * mean prob) = 1
    g.reset()
    s = SequenceLevelLoadBalanceLoss(1.0, 32)
    assert s(scores, idx, E, k).ndim == 0
    w = torch.ones(3, requires_grad=True)
    lb = (scores.sum() * 0 + scores[0, 0]) * 2
    out = MoELoadBalanceLossInjector.apply(w, lb)
    out.sum().backward()
    assert scores.grad[0, 0] == 2.0 and torch.equal(w.grad, torch.ones(3))


# ------------------------------------------------------------------------------------------------ MoE index math
def test_route_sort_ref_invariants():
    from pithtrain_b200.ops.moe import ALIGN, route_sort, sorted_capacity

    torch.manual_seed(0)
    n, k, E = 50, 3, 7
    eids = torch.randint(-1, E, (n, k), dtype=torch.int32)
    offs, ros, sor = route_sort(eids, E)
    assert sor.numel() == sorted_capacity(n * k, E)
    flat = eids.flatten()
    for e in range(E):
        a, b = int(offs[e]), int(offs[e + 1])
        assert (b - a) % ALIGN == 0
        slots = sor[a:b][sor[a:b] >= 0]
        assert torch.equal(flat[slots.long()], torch.full_like(slots, e))
        assert torch.equal(slots, slots.sort().values)  # stable: slot order inside a group
        assert slots.numel() == int((flat == e).sum())
    assert bool((ros[flat < 0] == -1).all())
    valid = flat >= 0
    assert torch.equal(sor[ros[valid].long()].long(), torch.nonzero(valid).flatten())


def test_ep_send_plan_index_math():
    from pithtrain_b200.parallel.ep import build_send_side

    torch.manual_seed(0)
    m, k, E, ep = 40, 4, 16, 4
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(m)]).int()
    tok, pos, eids, counts = build_send_side(idx, E, ep)
    epr = E // ep
    dest = idx.long() // epr
    assert counts.tolist() == [int((dest == g).any(1).sum()) for g in range(ep)]
    assert tok.numel() == int(counts.sum())
    for t in range(m):
        for g in range(ep):
            p = int(pos[t, g])
            if (dest[t] == g).any():
                assert int(tok[p]) == t
                row = eids[p]
                want = torch.where(dest[t] == g, idx[t].long() - g * epr, torch.full((k,), -1)).int()
                assert torch.equal(row, want)
            else:
                assert p == -1
    # expected de-duplicated volume under uniform routing
    exp = m * (1 - ((ep - 1) / ep) ** k)
    assert abs(float(counts.float().mean()) - exp) < 0.35 * exp


def test_moe_experts_cpu_vs_loop():
    from pithtrain_b200.ops import moe as M

    torch.manual_seed(0)
    n, k, E, H, I = 33, 2, 4, 16, 8
    x, w = torch.randn(n, H, requires_grad=True), torch.rand(n, k, requires_grad=True)
    eids = torch.stack([torch.randperm(E)[:k] for _ in range(n)]).int()
    eids[::5, 1] = -1
    w1, w2 = torch.randn(E, 2 * I, H) * 0.2, torch.randn(E, H, I) * 0.2
    b1, b2 = torch.nn.Parameter(torch.randn(E, 2 * I) * 0.1), torch.nn.Parameter(torch.randn(E, H) * 0.1)
    g1, g2 = torch.zeros_like(w1), torch.zeros_like(w2)
    for inter, limit in ((False, 0.0), (True, 7.0)):
        ew = M.ExpertWeights(w1, w2, lambda: g1, lambda: g2, b1=b1, b2=b2, interleaved=inter, alpha=1.702 if inter else 1.0, limit=limit)
        g1.zero_(); g2.zero_(); b1.grad = None; b2.grad = None
        x.grad = None; w.grad = None
        out = M.moe_experts(x, w, eids, ew)
        go = torch.randn(n, H)
        out.backward(go)
        got = (out.detach(), x.grad.clone(), w.grad.clone(), g1.clone(), g2.clone(), b1.grad.clone(), b2.grad.clone())
        leaves = [t.detach().clone().requires_grad_() for t in (x, w, w1, w2, b1, b2)]
        ref = M.moe_experts_ref(leaves[0], leaves[1], eids, leaves[2], leaves[3], leaves[4], leaves[5], inter, 1.702 if inter else 1.0, limit)
        ref.backward(go)
        want = (ref.detach(), leaves[0].grad, leaves[1].grad, leaves[2].grad, leaves[3].grad, leaves[4].grad, leaves[5].grad)
        for a, b in zip(got, want):
            assert torch.allclose(a, b, atol=1e-4, rtol=1e-4)


# ------------------------------------------------------------------------------------------------ data
def test_datasets(tmp_path):
    from pithtrain_b200.modules.dataset import ConcatDataset, MemmapDataset, SyntheticDataset

    for i, n in enumerate((41, 25)):
        with open(tmp_path / f"s{i}.bin", "wb") as f:
            np.save(f, (np.arange(n) + 100 * i).astype(np.uint16))
    a = MemmapDataset(tmp_path / "s0.bin", 8)
    assert len(a) == 5
    t, l = a[1]
    assert t.tolist() == list(range(8, 16)) and l.tolist() == list(range(9, 17))
    t, l = a.get_chunk(1, 2, 3)
    assert t.tolist() == [10, 11, 12] and l.tolist() == [11, 12, 13]
    c = ConcatDataset([a, MemmapDataset(tmp_path / "s1.bin", 8)], seed=3)
    assert len(c) == 8
    seen = sorted(int(c[i][0][0]) for i in range(8))
    assert seen == [0, 8, 16, 24, 32, 100, 108, 116]
    s = SyntheticDataset(1000, 16, seed=5)
    assert torch.equal(s[7][0], s[7][0]) and not torch.equal(s[7][0], s[8][0])
    assert torch.equal(s.get_chunk(7, 4, 4)[0], s[7][0][4:8]) and int(s[3][0].max()) < 1000


# ------------------------------------------------------------------------------------------------ native ABI table
def test_native_signature_table_matches_sources():
    from pithtrain_b200._native import SIGS

    src = "".join(open(f).read() for f in glob.glob(str(ROOT / "pithtrain_b200" / "csrc" / "*.cu")))
    found = 0
    for m in re.finditer(r"PT_API int (\w+)\(([^)]*)\)", src):
        name, args = m.group(1), [a.strip() for a in m.group(2).split(",") if a.strip()]
        sig = "".join("P" if "*" in a else "L" if a.startswith("long long") else "F" if a.startswith("float") else "I" for a in args)
        assert name in SIGS, f"{name} is exported but has no ctypes signature"
        assert SIGS[name] == sig, (name, SIGS[name], sig)
        found += 1
    assert found >= 30


def test_reference_package_name_alias():
    """Scripts written against the reference's package name import this framework's modules."""
    from pithtrain.modules.training import make_muon_optimizer, make_wsd_scheduler  # noqa: F401
    from pithtrain.operators.ring_attention import ring_attention_func
    from pithtrain.tasks.pretrain_lm import PretrainLMCfg, launch  # noqa: F401

    import pithtrain_b200.ops.ring_attention as impl
    import pithtrain_b200.tasks.pretrain_lm as impl_task

    assert ring_attention_func is impl.ring_attention_func and PretrainLMCfg is impl_task.PretrainLMCfg
    import pithtrain.contexts.distributed as ctx_alias
    import pithtrain_b200.contexts.distributed as ctx_impl

    assert ctx_alias is ctx_impl  # one module object: no duplicated global state


@pytest.mark.parametrize("window,use_sinks,packed", [(127, True, False), (128, False, True), (5, True, True), (200, False, False)])
def test_blocked_sliding_window_attention(window, use_sinks, packed):
    from pithtrain_b200.ops.attention import attention, attention_ref, attention_window_blocked, segments_from_cu_seqlens

    torch.manual_seed(0)
    B, S, Hq, Hkv, D = 2, 512, 4, 2, 16
    q, k, v = [torch.randn(B, S, h, D, requires_grad=True) for h in (Hq, Hkv, Hkv)]
    sinks = torch.randn(Hq, requires_grad=True) if use_sinks else None
    cu = torch.tensor([0, 100, 300, S], dtype=torch.int32) if packed else None
    ref = attention_ref(q, k, v, True, None, window, sinks, cu)
    seg = segments_from_cu_seqlens(cu, S) if packed else None
    out = attention_window_blocked(q, k, v, window, None, sinks, seg)
    leaves = [q, k, v] + ([sinks] if use_sinks else [])
    go = torch.randn_like(ref)
    for a, b in zip((ref,) + torch.autograd.grad(ref, leaves, go), (out,) + torch.autograd.grad(out, leaves, go)):
        assert torch.allclose(a, b, atol=2e-5, rtol=1e-4)
    if S > 2 * (window + 128):  # the public entry point picks the blocked form by itself
        assert torch.allclose(attention(q, k, v, True, None, window, sinks, cu), ref, atol=2e-5, rtol=1e-4)


def test_own_attention_predicate_and_row_bounds():
    """The kernels' predicate refuses CPU tensors, fp32 and head dims outside their set; the per-row lower key bounds
    fold sliding windows and document starts into one vector."""
    from pithtrain_b200.ops import attention_native as N

    q = torch.zeros(2, 256, 8, 128, dtype=torch.bfloat16)
    k = v = torch.zeros(2, 256, 2, 128, dtype=torch.bfloat16)
    assert not N.supported(q, k, v, True, None, None, None)  # CPU tensors never take the kernels
    assert N.row_lower_bounds(2, 256, 0, None, None, "cpu") is None
    lo = N.row_lower_bounds(1, 8, 0, 2, None, "cpu")
    assert lo.tolist() == [0, 0, 0, 1, 2, 3, 4, 5]
    lo = N.row_lower_bounds(1, 8, 4, 2, None, "cpu")  # queries 4 positions ahead of key 0
    assert lo.tolist() == [2, 3, 4, 5, 6, 7, 8, 9]
    cu = torch.tensor([0, 3, 8], dtype=torch.int32)
    assert N.row_lower_bounds(1, 8, 0, None, cu, "cpu").tolist() == [0, 0, 0, 3, 3, 3, 3, 3]
    assert N.row_lower_bounds(1, 8, 0, 1, cu, "cpu").tolist() == [0, 0, 1, 3, 3, 4, 5, 6]
    assert N.row_lower_bounds(2, 4, 0, 1, None, "cpu").tolist() == [0, 0, 1, 2, 0, 0, 1, 2]


@pytest.mark.parametrize("shape", [(3, 64, 128), (2, 128, 64), (64, 64), (1, 192, 64)])
def test_newton_schulz_on_grouped_gemm_products_matches_batched(shape):
    """The formulation on M-/K-grouped GEMMs (wide and tall, stacks and single matrices) is the same iteration."""
    from pithtrain_b200.modules.optimizer import newtonschulz5_own_gemm, zeropower_via_newtonschulz5

    torch.manual_seed(3)
    G = torch.randn(*shape)
    got = newtonschulz5_own_gemm(G).float()
    want = zeropower_via_newtonschulz5(G).float()
    assert got.shape == want.shape
    # two bf16 evaluations of the same polynomial (A^2 is rounded before it is combined here, after there)
    assert float((got - want).abs().max()) < 0.06 and float((got - want).norm() / want.norm()) < 0.05
    sv = torch.linalg.svdvals(got)
    assert float(sv.max()) < 1.5
    if shape[-1] != shape[-2]:  # a square Gaussian matrix has singular values near zero that five steps cannot lift
        assert float(sv.min()) > 0.5
    U, _, Vh = torch.linalg.svd(G.float(), full_matrices=False)
    polar = U @ Vh
    assert float((got * polar).sum() / (got.norm() * polar.norm())) > 0.97


def test_native_call_sites_match_the_signature_table():
    """Every ``.pt_*(...)`` call in the Python sources names an entry of ``_native.SIGS`` and passes as many arguments
    as the entry declares; the built library (when present) exports every entry. ctypes would otherwise only complain
    when the call is reached, which for most of them is on a GPU."""
    import ast
    import ctypes

    from pithtrain_b200 import _native

    files = [p for root in ("pithtrain_b200", "benchmarks", "tests") for p in (ROOT / root).rglob("*.py")]
    files += [ROOT / "bench.py", ROOT / "__graft_entry__.py"]
    problems = []
    for path in files:
        for node in ast.walk(ast.parse(path.read_text())):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr.startswith("pt_")):
                continue
            name = node.func.attr
            if name not in _native.SIGS:
                problems.append(f"{path.name}:{node.lineno}: {name} is not in SIGS")
            elif not any(isinstance(a, ast.Starred) for a in node.args) and len(node.args) != len(_native.SIGS[name]):
                problems.append(f"{path.name}:{node.lineno}: {name} called with {len(node.args)} arguments, SIGS declares {len(_native.SIGS[name])}")
    assert not problems, problems
    lib = ROOT / "pithtrain_b200" / "_lib" / "libpithb200.so"
    if lib.exists():
        handle = ctypes.CDLL(str(lib))
        assert not [n for n in _native.SIGS if not hasattr(handle, n)]


def test_channel_struct_layouts_match_the_library():
    """The ctypes mirrors of the channel structs that kernels take by value have the size the compiled library reports
    (host-only functions, so the check runs without a GPU)."""
    import ctypes

    lib = ROOT / "pithtrain_b200" / "_lib" / "libpithb200.so"
    if not lib.exists():
        pytest.skip("native library not built")
    handle = ctypes.CDLL(str(lib))
    from pithtrain_b200.parallel.ep_fused import EpChanStruct
    from pithtrain_b200.parallel.fsdp_fused import FsdpChanStruct

    assert ctypes.sizeof(EpChanStruct) == handle.pt_ep_chan_struct_size()
    assert ctypes.sizeof(FsdpChanStruct) == handle.pt_fsdp_chan_struct_size()


@pytest.mark.parametrize("S,chunk", [(64, 64), (100, 32), (7, 64), (130, 64)])
def test_gated_delta_rule_chunked_equals_the_recurrence(S, chunk):
    """Chunked evaluation (triangular solve inside a chunk, state carried across chunks) against the token-by-token
    recurrence, outputs and every input gradient, for lengths that are and are not multiples of the chunk."""
    from pithtrain_b200.ops.gated_delta_rule import gated_delta_rule, gated_delta_rule_recurrent

    torch.manual_seed(4)
    B, H, dk, dv = 2, 3, 8, 6
    q, k = torch.randn(B, S, H, dk), torch.nn.functional.normalize(torch.randn(B, S, H, dk), dim=-1)
    v = torch.randn(B, S, H, dv)
    g = -torch.rand(B, S, H) * 0.5  # log decay <= 0
    beta = torch.rand(B, S, H)
    go = torch.randn(B, S, H, dv)
    outs = []
    for fn in (lambda *a: gated_delta_rule(*a, chunk_size=chunk), gated_delta_rule_recurrent):
        leaves = [t.clone().requires_grad_() for t in (q, k, v, g, beta)]
        o = fn(*leaves)
        o.backward(go)
        outs.append((o.detach(), [t.grad for t in leaves]))
    (o1, g1), (o2, g2) = outs
    assert torch.allclose(o1, o2, atol=2e-4, rtol=1e-4), float((o1 - o2).abs().max())
    for a, b in zip(g1, g2):
        assert torch.allclose(a, b, atol=5e-4, rtol=1e-3), float((a - b).abs().max())


def test_new_entry_points_validate_their_arguments_on_the_host():
    """Shape errors are refused with -2 before any CUDA call; valid shapes get as far as the tensor-map encoder, which
    has no driver here and reports -3 — neither path launches or crashes without a GPU."""
    import ctypes

    from pithtrain_b200 import _native

    lib = ROOT / "pithtrain_b200" / "_lib" / "libpithb200.so"
    if not lib.exists():
        pytest.skip("native library not built")
    if torch.cuda.is_available():
        pytest.skip("host-only check")
    L = ctypes.CDLL(str(lib))
    for name in ("pt_attn_fwd", "pt_attn_bwd", "pt_gemm2cta_nt"):
        fn = getattr(L, name)
        fn.argtypes = [_native._CT[a] for a in _native.SIGS[name]]
        fn.restype = ctypes.c_int
    N = None
    fwd = lambda Sq, Sk, Hq, Hkv, dqk, dv: L.pt_attn_fwd(N, N, N, N, N, N, N, 1, Sq, Sk, Hq, Hkv, dqk, dv, Hq * dqk, Hkv * dqk,
                                                         Hkv * dv, Hq * dv, 0.1, 1, 0, N)
    assert fwd(256, 256, 5, 2, 128, 128) == -2  # heads not divisible
    assert fwd(256, 0, 4, 2, 128, 128) == -2    # no keys
    assert fwd(256, 256, 4, 2, 96, 96) == -2    # head dim outside the kernels' set
    assert fwd(256, 128, 4, 2, 128, 128) == -3
    bwd = lambda Sq, Hq, Hkv, dd: L.pt_attn_bwd(N, N, N, N, N, N, N, N, N, N, N, N, N, N, N, 1, Sq, Sq, Hq, Hkv, dd, Hq * dd,
                                                Hkv * dd, Hkv * dd, Hq * dd, Hq * dd, 0.1, 1, 0, N)
    assert bwd(256, 5, 2, 128) == -2
    assert bwd(256, 4, 2, 192) == -2            # the backward covers head dims 64 and 128
    assert bwd(256, 4, 2, 128) == -3
    assert L.pt_gemm2cta_nt(N, N, N, 256, 256, 60, 60, 60, 256, N) == -2  # K not a multiple of 8
    assert L.pt_gemm2cta_nt(N, N, N, 256, 256, 64, 64, 64, 256, N) == -3


def test_bounds_checking_variant_compiles():
    """``-DPT_BOUNDS_CHECK`` turns the index validation of the peer-memory exchange kernels on; the variant must keep
    compiling for sm_100a (the regular build compiles the checks away)."""
    import shutil
    import subprocess
    import tempfile

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("no nvcc")
    from pithtrain_b200 import build as B

    src = ROOT / "pithtrain_b200" / "csrc" / "ep_fused.cu"
    with tempfile.TemporaryDirectory() as d:
        res = subprocess.run([nvcc, *B.NVCC_FLAGS, "-DPT_BOUNDS_CHECK", "-c", str(src), "-o", str(Path(d) / "x.o")],
                             capture_output=True, text=True)
        assert res.returncode == 0, res.stderr[-2000:]
    assert "PT_IN_BOUNDS" in src.read_text()
