"""The Rososun design in the engine against the plain numpy statement of it (tests/plain/rososun_plain.py).

Every test makes its own small configuration and random weights.  Each body runs twice: with the PyTorch
stand-ins for the kernels on the CPU (the parts, the cache manager, the batching), and on the GPU with the
real kernels (marked ``gpu``).  Sizes differ from one another in everything a configuration can say: widths
that are no multiple of heads x dim, value sizes unlike key sizes, several norm groups or one, layers without
a feed-forward, layers that use another layer's tensors.
"""

import json
import os

import numpy as np
import pytest
import torch

from tests import traces
from tests.plain import rososun_plain as plain

DELTA = {"heads": 2, "dim": 32, "decay_rank": 6}
CONFIG_A = {
    "architecture": "Rososun", "vocab": 320, "width": 96, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6, "groups": 3},
    "layers": [
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "vdim": 24, "kv_rank": 40, "scale": 0.2},
         "mlp": {"kind": "dense", "ff": 160}},
        {"type": "general_delta", "mixer": DELTA, "mlp": {"kind": "dense", "ff": 112}},
        {"type": "general_delta", "mixer": DELTA, "mlp": {"kind": "dense", "ff": 112}, "weights_of": 1},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 32, "vdim": 16, "kv_rank": 24, "scale": 0.15}, "mlp": None},
    ],
}
LATENT_B = {"heads": 4, "dim": 16, "vdim": 16, "kv_rank": 64, "scale": 0.3}
CONFIG_B = {          # one norm group, one head in the recurrent layer, a latent of a size the tensor-core kernels take
    "architecture": "Rososun", "vocab": 200, "width": 128, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5, "groups": 1},
    "layers": [
        {"type": "general_delta", "mixer": {"heads": 1, "dim": 48, "decay_rank": 9}, "mlp": None},
        {"type": "latent_attention", "mixer": LATENT_B, "mlp": {"kind": "dense", "ff": 200}},
        {"type": "latent_attention", "mixer": LATENT_B, "mlp": {"kind": "dense", "ff": 200}, "weights_of": 1},
        {"type": "general_delta", "mixer": {"heads": 5, "dim": 16, "decay_rank": 3}, "mlp": {"kind": "dense", "ff": 72}},
    ],
}
CONFIG_C = {          # many heads over latents of the sizes the tensor-core attention kernels take: 16, 32 and 8 heads share one latent
    "architecture": "Rososun", "vocab": 260, "width": 192, "embedding": {"scale": 9.0}, "norm": {"eps": 1e-5, "groups": 2},
    "layers": [
        {"type": "latent_attention", "mixer": {"heads": 16, "dim": 16, "vdim": 8, "kv_rank": 128, "scale": 0.25}, "mlp": {"kind": "dense", "ff": 256}},
        {"type": "general_delta", "mixer": {"heads": 3, "dim": 64, "decay_rank": 8}, "mlp": {"kind": "dense", "ff": 256}},
        {"type": "latent_attention", "mixer": {"heads": 32, "dim": 8, "vdim": 8, "kv_rank": 32, "scale": 0.35}, "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 8, "dim": 24, "vdim": 24, "kv_rank": 16, "scale": 0.2}, "mlp": {"kind": "dense", "ff": 64}},
        # 24 heads on one latent of 64: even a single decoded token is more rows than the decode form's tile takes
        {"type": "latent_attention", "mixer": {"heads": 24, "dim": 8, "vdim": 8, "kv_rank": 64, "scale": 0.3}, "mlp": None},
    ],
}
ONLY_DELTA = {"architecture": "Rososun", "vocab": 90, "width": 64, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6, "groups": 2},
              "layers": [{"type": "general_delta", "mixer": {"heads": 2, "dim": 24, "decay_rank": 4}, "mlp": {"kind": "dense", "ff": 96}},
                         {"type": "general_delta", "mixer": {"heads": 2, "dim": 24, "decay_rank": 4}, "mlp": {"kind": "dense", "ff": 96}, "weights_of": 0}]}
ONLY_LATENT = {"architecture": "Rososun", "vocab": 90, "width": 64, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6, "groups": 8},
               "layers": [{"type": "latent_attention", "mixer": {"heads": 2, "dim": 16, "vdim": 20, "kv_rank": 12, "scale": 0.3}, "mlp": None}]}
ODD = {               # sizes that are multiples of nothing: no 16-byte row anywhere, so every kernel's plain form runs
    "architecture": "Rososun", "vocab": 77, "width": 50, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-4, "groups": 5},
    "layers": [{"type": "general_delta", "mixer": {"heads": 3, "dim": 12, "decay_rank": 5}, "mlp": {"kind": "dense", "ff": 54}},
               {"type": "latent_attention", "mixer": {"heads": 3, "dim": 10, "vdim": 14, "kv_rank": 21, "scale": 0.4}, "mlp": {"kind": "dense", "ff": 54}}]}
CONFIGS = {"A": (CONFIG_A, 16), "B": (CONFIG_B, 8), "C": (CONFIG_C, 16), "only_delta": (ONLY_DELTA, 4), "only_latent": (ONLY_LATENT, 32),
           "odd": (ODD, 16)}


def _devices():
    return [pytest.param("cpu", id="stand-in"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]


@pytest.fixture(params=_devices())
def dev(request):
    """The device a body runs on; on the CPU the PyTorch stand-ins take the kernels' place."""
    if request.param == "cpu":
        request.getfixturevalue("cpu_ops")
    elif not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return request.param


def make_model(tmp_path, config, seed=5, name="m", edit=None, std=0.08):
    """A model folder from the configuration and a seed.  ``edit(tensors)`` may change the drawn tensors (float32
    numpy arrays by name) before they are written."""
    from sllm_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    d = write_random_model(os.path.join(str(tmp_path), name), config, seed, std=std, bias_std=0.3, gain_std=0.2)
    if edit is not None:
        f = SafetensorsFile(os.path.join(d, "model.safetensors"))
        t = {n: f.tensor(n).float() for n in f.names()}
        edit(t)
        del f
        write_safetensors(os.path.join(d, "model.safetensors"), {n: v.to(torch.bfloat16) for n, v in t.items()})
    return d


def plain_logits(d, reqs):
    cfg, w = plain.load_model(d)
    return {r: plain.forward(ids, cfg, w).astype(np.float32) for r, ids in reqs.items()}


def compare(tr, out, want, dtype, what):
    """float32: every logit to 2e-4.  bfloat16: the difference of a row (mean taken off, root mean square over the
    vocabulary) relative to the row's own spread is rounding's: under 2 % for 19 rows in 20 and under 8 % for every row
    (measured: median 0.4 %, the worst row 3.4 %; a lost key or state moves rows by tens of per cent)."""
    if dtype == "float32":
        return traces.compare(tr, out, want, what=what, rtol=2e-4, atol=2e-4)
    errs = []
    for s in tr.steps:
        for row, (req, pos) in enumerate(s["expect"]):
            ref, got = want[req][pos], out[s["step"]][row]
            d, r = got - ref, ref - ref.mean()
            e = float(np.sqrt(((d - d.mean()) ** 2).mean()) / np.sqrt((r ** 2).mean()))
            assert e < 0.08, f"{what}: step {s['step']}, request {req!r}, position {pos}: relative difference {e:.3g}"
            errs.append(e)
    assert np.quantile(errs, 0.95) < 0.02, f"{what}: 95th percentile of the rows' relative difference {np.quantile(errs, 0.95):.3g}"


def dtypes_on(dev):
    return ("float32",) if dev == "cpu" else ("float32", "bfloat16")


# ---- configuration, plan, weights ---------------------------------------------------------------------------

def test_config_plan_and_cache_needs():
    from sllm_b200.config import ConfigError, architecture_of
    from sllm_b200.models.causal_lm import CausalLM
    from sllm_b200.parts import PagedKV, SlotState
    arch = architecture_of(CONFIG_A)
    cfg = arch.config_cls.from_dict(CONFIG_A)
    assert cfg.to_dict() == CONFIG_A
    p = arch.plan(cfg)
    assert [e.layer for e in p.run_list] == [0, 1, 1, 2] and len(p.layers) == 3 and p.embedding_scale == 4.0
    assert "ffn" not in p.layers[2].parts
    m = CausalLM(p, dtype=torch.float32, device="cpu")
    needs = [n for _, n in m.cache_needs()]
    assert needs[0] == (PagedKV(1, 40, None, values=False), SlotState((96,), "shift"))
    assert needs[1] == needs[2] == (SlotState((2, 32, 32), "delta"), SlotState((96,), "shift"))
    names = {s.name for s in m.tensor_specs()}
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.shift", "l0.mix.dkv.norm", "l1.mix.a.b", "l1.mlp.down.b", "l3.mix.g"} <= names
    assert not any(n.startswith("l2.") or n.startswith("l3.mlp") for n in names)
    for bad in (dict(CONFIG_A, width=97), dict(CONFIG_A, norm={"eps": 1e-6, "groups": 5}),
                dict(CONFIG_A, layers=[dict(CONFIG_A["layers"][0], type="other")]),
                dict(CONFIG_A, layers=[CONFIG_A["layers"][0], dict(CONFIG_A["layers"][1], weights_of=0)]),
                {k: v for k, v in CONFIG_A.items() if k != "embedding"}):
        with pytest.raises(ConfigError):
            arch.config_cls.from_dict(bad)


def test_decay_rank_is_read_from_the_checkpoint(tmp_path):
    """A size that config.json does not give is taken from the tensor's shape; a pair that disagrees is refused."""
    from sllm_b200.engine import build_model
    d = make_model(tmp_path, CONFIG_A)
    with open(os.path.join(d, "config.json")) as f:
        raw = json.load(f)
    for layer in raw["layers"]:
        layer["mixer"].pop("decay_rank", None)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(raw, f)
    model, _ = build_model(d, "float32", "cpu")
    assert model.layers[1].mixer.rank == 6


# ---- each mechanism alone: an operation against the plain function ---------------------------------------------------

def _step(dev, q_lens, slots):
    from sllm_b200.parts import StepContext
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    starts = np.concatenate([[0], np.cumsum(q_lens)])
    return StepContext(num_tokens=int(starts[-1]), num_seqs=len(q_lens), token_ids=i32([0] * int(starts[-1])),
                       positions=i32([0] * int(starts[-1])), seq_of_token=i32(np.repeat(np.arange(len(q_lens)), q_lens).tolist()),
                       q_start=i32(starts.tolist()), ctx_len=i32(q_lens), state_slots=i32(slots), logit_rows=i32([]), groups=[],
                       q_lens=list(q_lens), ctx_lens=list(q_lens), max_q_len=max(q_lens), max_ctx_len=max(q_lens))


def test_sinusoid_and_scaled_embedding(dev):
    import sllm_b200.ops as ops
    rng = np.random.default_rng(0)
    W, V = 48, 30
    table = torch.from_numpy(rng.standard_normal((V, W)).astype(np.float32)).to(dev)
    ids = rng.integers(0, V, 9)
    pos = np.array([0, 1, 2, 3, 700, 701, 5, 65000, 12])
    x = ops.embed_gather(table, torch.tensor(ids, dtype=torch.int32, device=dev), 3.5)
    f = torch.from_numpy((10000.0 ** (-2.0 * np.arange(W // 2) / W)).astype(np.float32)).to(dev)
    ops.add_sinusoid_(x, torch.tensor(pos, dtype=torch.int32, device=dev), f)
    want = plain.embedding(ids, table.cpu().numpy().astype(np.float64), 3.5) + plain.sinusoid(pos, W, np.float32)
    np.testing.assert_allclose(x.cpu().numpy(), want, atol=3e-6 * 65000 / 1000 + 1e-5)      # (a float32 angle near 65000 is exact to ~4e-3)
    np.testing.assert_allclose(x.cpu().numpy()[:4], want[:4], atol=1e-5)


@pytest.mark.parametrize("groups", [1, 4, 6, 16])
def test_group_norm_with_pending_terms_and_token_shift_across_portions(dev, groups):
    import sllm_b200.ops as ops
    rng = np.random.default_rng(groups)
    W, eps = 48, 1e-5
    lens = [5, 1, 2, 7]                     # four requests in one batch
    T = sum(lens)
    x = rng.standard_normal((T, W)) * 3
    t0, t1 = rng.standard_normal((T, W)), rng.standard_normal((2, T, W))
    gain, mix = 1 + 0.3 * rng.standard_normal(W), rng.uniform(0, 1, W)
    before = rng.standard_normal((6, W))    # the state slots' content: each request's previous normed row
    slots = [4, 0, 3, 1]
    to = lambda a: torch.from_numpy(np.asarray(a, dtype=np.float32)).to(dev).contiguous()
    stream, state = to(x), to(before)
    rinv = ops.add_group_ssq(stream, [to(t0), to(t1)], groups, eps)
    full = x + t0 + t1.sum(0)
    np.testing.assert_allclose(stream.cpu().numpy(), full, rtol=1e-6, atol=1e-5)
    h, hs = ops.group_norm_shift(stream, rinv, to(gain), torch.float32, mix=to(mix), state=state, step=_step(dev, lens, slots))
    want_h = plain.group_norm(full, gain, groups, eps)
    np.testing.assert_allclose(h.cpu().numpy(), want_h, rtol=2e-5, atol=2e-5)
    at = 0
    for n, slot in zip(lens, slots):
        want = plain.token_shift(want_h[at:at + n], mix, before[slot])
        np.testing.assert_allclose(hs.cpu().numpy()[at:at + n], want, rtol=2e-5, atol=2e-5)
        np.testing.assert_allclose(state.cpu().numpy()[slot], want_h[at + n - 1], rtol=2e-5, atol=2e-5)   # the slot now holds the last row
        at += n
    np.testing.assert_allclose(state.cpu().numpy()[[2, 5]], before[[2, 5]], rtol=1e-6)                   # slots of nobody stay
    only = ops.group_norm_shift(stream, rinv, to(gain), torch.float32)
    np.testing.assert_allclose(only.cpu().numpy(), want_h, rtol=2e-5, atol=2e-5)
    # the same with the reciprocal roots taken by the kernel itself, from fresh slots
    state2 = to(before)
    h2, hs2 = ops.group_norm_shift(stream, None, to(gain), torch.float32, groups=groups, eps=eps, mix=to(mix), state=state2,
                                   step=_step(dev, lens, slots))
    np.testing.assert_allclose(h2.cpu().numpy(), want_h, rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(hs2.cpu().numpy(), hs.cpu().numpy(), rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(state2.cpu().numpy(), state.cpu().numpy(), rtol=2e-5, atol=2e-5)


def test_gated_activation(dev):
    import sllm_b200.ops as ops
    rng = np.random.default_rng(1)
    gu = rng.standard_normal((7, 2 * 36)) * 3
    t = torch.from_numpy(gu.astype(np.float32)).to(dev)
    got = ops.act_mul(t, 36, torch.float32, "gelu_tanh").cpu().numpy()
    np.testing.assert_allclose(got, plain.gelu_tanh(gu[:, :36]) * gu[:, 36:], rtol=1e-5, atol=1e-5)
    got = ops.act_mul(t, 36, torch.float32, "silu").cpu().numpy()
    np.testing.assert_allclose(got, gu[:, :36] * plain.sigmoid(gu[:, :36]) * gu[:, 36:], rtol=1e-5, atol=1e-5)
    got = ops.tanh_cols(t, 5, 11, torch.float32).cpu().numpy()
    np.testing.assert_allclose(got, np.tanh(gu[:, 5:16]), rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,I", [(5, 128, 200), (32, 256, 384), (200, 128, 200), (300, 256, 1024), (64, 256, 384), (7, 96, 40)])
def test_gated_feed_forward_product_with_its_activation_in_the_epilogue(M, K, I):
    """gelu_tanh(x Wg^T + bg) * (x Wu^T + bu) from the kernels that apply it as the product's tile leaves (few tokens: the
    streaming kernel; a prompt portion: the CTA-pair product) and from the product followed by the activation kernel,
    against float64; sizes that take each path, and one that no fused form takes."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import sllm_b200.ops as ops
    rng = np.random.default_rng(M + K)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda().to(torch.bfloat16)
    wg, wu = (torch.from_numpy((rng.standard_normal((I, K)) * 0.2).astype(np.float32)).cuda().to(torch.bfloat16) for _ in range(2))
    bg, bu = (torch.from_numpy(rng.standard_normal(I).astype(np.float32)).cuda() for _ in range(2))
    xd = x.double().cpu().numpy()
    want = plain.gelu_tanh(xd @ wg.double().cpu().numpy().T + bg.double().cpu().numpy()) * (xd @ wu.double().cpu().numpy().T + bu.double().cpu().numpy())
    n = 8 if I % 8 == 0 else I
    alt = lambda a, c: torch.stack([a.reshape(I // n, n, *a.shape[1:]), c.reshape(I // n, n, *c.shape[1:])], dim=1).reshape(2 * I, *a.shape[1:]).contiguous()
    before = dict(ops.launches)
    got = ops.linear_act_mul(x, alt(wg, wu), alt(bg, bu), n, torch.bfloat16, "gelu_tanh").float().cpu().numpy()
    fused = ops.stream_supports(M, 2 * I, K) or (M > 128 and ops.pair_supports(M, 2 * I, K))
    # (the unfused form rounds gate and up to bfloat16 before the activation: one rounding more, of values up to 16)
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=3e-2 if fused else 1e-1)
    assert (ops.launches["own"] + ops.launches["library"] - before["own"] - before["library"] == 1) == bool(fused and n == 8 and (2 * I) % 16 == 0)
    ops.check_tcgen05_status()


@pytest.mark.parametrize("heads,dk", [(1, 64), (3, 16), (2, 40), (1, 130), (80, 16), (2, 6)])
def test_delta_rule_recurrence_in_portions_and_slots(dev, heads, dk):
    """The recurrence alone: two requests side by side, each cut into portions (down to one token) that continue from
    the state slot, against the whole sequences through the plain recurrence."""
    import sllm_b200.ops as ops
    rng = np.random.default_rng(dk)
    C = heads * dk
    lens = {0: 37, 1: 21}
    R = 4
    w = {f"m.{n}": rng.standard_normal((C, C)) * 0.3 for n in ("r", "k", "v", "g", "a")}
    w.update({"m.w1": rng.standard_normal((R, C)) * 0.3, "m.w2": rng.standard_normal((C, R)), "m.w0": rng.standard_normal(C) - 2.0,
              "m.a.b": rng.standard_normal(C), "m.norm": 1 + 0.2 * rng.standard_normal(C), "m.o": np.eye(C)})
    xs = {s: rng.standard_normal((n, C)) for s, n in lens.items()}
    want = {s: plain.general_delta(x, w, "m", heads, dk, 1e-5) for s, x in xs.items()}
    to = lambda a: torch.from_numpy(np.asarray(a, dtype=np.float32)).to(dev).contiguous()
    state = torch.zeros((3, heads, dk, dk), dtype=torch.float32, device=dev)
    slots = {0: 2, 1: 0}
    got = {s: [] for s in lens}
    at = {s: 0 for s in lens}
    cuts = [(17, 1), (1, 2), (2, 9), (13, 1), (4, 8)]
    for c in cuts:
        live = [s for s in lens if at[s] < lens[s]]
        q = [min(c[s], lens[s] - at[s]) for s in live]
        x = np.concatenate([xs[s][at[s]:at[s] + n] for s, n in zip(live, q)])
        cols = np.concatenate([x @ w[f"m.{n}"].T for n in ("r", "k", "v", "a", "g")], axis=1)
        decay = np.tanh(x @ w["m.w1"].T) @ w["m.w2"].T + w["m.w0"]
        proj = to(cols)
        o = ops.delta_rule(proj, (0, C, 2 * C, 3 * C), to(decay), to(w["m.a.b"]), state, _step(dev, q, [slots[s] for s in live]), heads, dk, dk)
        y = ops.delta_out(o, to(w["m.norm"]), proj, 4 * C, 1e-5, heads, dk, torch.float32).cpu().numpy()
        r0 = 0
        for s, n in zip(live, q):
            got[s].append(y[r0:r0 + n])
            r0 += n
            at[s] += n
    assert all(at[s] == lens[s] for s in lens)
    for s in lens:
        np.testing.assert_allclose(np.concatenate(got[s]), want[s][0], rtol=3e-4, atol=3e-4)
        np.testing.assert_allclose(state[slots[s]].cpu().numpy(), want[s][1], rtol=3e-4, atol=3e-4)
    assert float(state[1].abs().max()) == 0.0


def test_head_products_and_latent_write(dev):
    import sllm_b200.ops as ops
    rng = np.random.default_rng(2)
    T, H, din, dout, ld = 70, 3, 20, 24, 100
    x = rng.standard_normal((T, ld))
    w = rng.standard_normal((H, dout, din))
    to = lambda a: torch.from_numpy(np.asarray(a, dtype=np.float32)).to(dev).contiguous()
    got = ops.head_linear(to(x), 7, to(w), torch.float32, gate=to(x), goff=80).cpu().numpy()
    want = np.einsum("thi,hoi->tho", x[:, 7:7 + H * din].reshape(T, H, din), w) * plain.sigmoid(x[:, 80:80 + H])[:, :, None]
    np.testing.assert_allclose(got, want.reshape(T, H * dout), rtol=1e-4, atol=1e-4)
    # bfloat16 operands (the tensor-core form on the GPU): x in float32 or bfloat16, rows that allow 16-byte loads and
    # rows that do not, sizes that end inside a tile
    for T2, H2, din2, dout2, xoff2 in ((70, 3, 20, 24, 7), (150, 2, 64, 96, 8), (9, 5, 128, 40, 0)):
        ld2 = xoff2 + H2 * din2 + 16
        x2 = rng.standard_normal((T2, ld2))
        w2 = rng.standard_normal((H2, dout2, din2)) * 0.3
        wb = to(w2).to(torch.bfloat16)
        for xt in (to(x2), to(x2).to(torch.bfloat16)):
            got = ops.head_linear(xt, xoff2, wb, torch.bfloat16, gate=to(x2), goff=ld2 - H2).float().cpu().numpy()
            xs = xt.to(torch.bfloat16).double().cpu().numpy()[:, xoff2:xoff2 + H2 * din2].reshape(T2, H2, din2)
            want = np.einsum("thi,hoi->tho", xs, wb.double().cpu().numpy()) * plain.sigmoid(x2[:, ld2 - H2:])[:, :, None]
            np.testing.assert_allclose(got, want.reshape(T2, H2 * dout2), rtol=1e-2, atol=1e-2)
    rank, ps = 24, 4
    cache = torch.zeros((30, 1, ps, rank), dtype=torch.float32, device=dev)
    gain = 1 + 0.2 * rng.standard_normal(rank)
    slots = rng.permutation(30 * ps)[:T].astype(np.int32)
    slots[5] = -1                        # a row that pads a batch writes nothing
    ops.latent_write(to(x), 33, rank, to(gain), 1e-5, torch.from_numpy(slots).to(dev), cache)
    c = plain.unit_rms(x[:, 33:33 + rank], 1e-5) * gain
    flat = cache.cpu().numpy().reshape(30 * ps, rank)
    keep = slots >= 0
    np.testing.assert_allclose(flat[slots[keep]], c[keep], rtol=2e-5, atol=2e-5)
    untouched = np.setdiff1d(np.arange(30 * ps), slots[keep])
    assert not flat[untouched].any()


# ---- the whole model through the engine: every cutting against the plain implementation ---------------------------

def _requests(vocab, lengths, seed=3):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, vocab, n).tolist() for i, n in enumerate(lengths)}


@pytest.mark.parametrize("which", ["A", "B", "C", "only_delta", "only_latent", "odd"])
def test_every_cutting_against_plain(tmp_path, dev, which):
    """Whole prompts; most of a prompt and the rest token by token; portions of changing size down to two tokens;
    up to four requests at a time, portions beside single tokens.  The pools hold the trace's peak only and freed pages
    are poisoned, so pages and state slots are used again and a read of a page no longer held would show."""
    from sllm_b200.engine import Engine, build_model
    config, page = CONFIGS[which]
    d = make_model(tmp_path, config)
    reqs = _requests(config["vocab"], (70, 37, 100, 1, 45, 64, 23))
    want = plain_logits(d, reqs)
    for dtype in dtypes_on(dev):
        model, _ = build_model(d, dtype, dev)
        for mode in ("whole", "tail_decode", "portions", "mixed"):
            tr = getattr(traces, mode)(reqs)
            eng = Engine(model, page_size=page, num_pages=tr.max_tokens // page, max_requests=4, poison_freed=True)
            out = traces.replay_engine(tr, eng)
            compare(tr, out, want, dtype, f"{which}/{dtype}/{mode}")
            eng.cache.check()
            assert not eng.cache.requests and all(g.pool.used_count == 0 for g in eng.cache.groups)
            if mode == "mixed" and eng.cache.groups:
                assert eng.cache.reuse_count > 0


def test_batch_of_unequal_requests_equals_each_alone(tmp_path, dev):
    """The same tokens alone and in a batch of unequal requests, in different state slots and pages: the logits agree to
    rounding (in float32, to 1e-5)."""
    from sllm_b200.engine import Engine, StepEntry, build_model
    d = make_model(tmp_path, CONFIG_A)
    reqs = _requests(CONFIG_A["vocab"], (33, 2, 19, 50), seed=8)
    model, _ = build_model(d, "float32", dev)
    alone = {}
    for r, ids in reqs.items():
        eng = Engine(model, page_size=16, num_pages=8, max_requests=2)
        a = eng.step([StepEntry(r, ids[:-1], [len(ids) - 2])])
        b = eng.step([StepEntry(r, ids[-1:], [0])])
        alone[r] = torch.cat([a, b]).cpu().numpy()
    eng = Engine(model, page_size=16, num_pages=16, max_requests=5)
    eng.step([StepEntry("warm", [1, 2, 3], [])])            # takes slot 0 and the first page, then leaves
    eng.finish("warm")
    order = ["r3", "r1", "r0", "r2"]
    a = eng.step([StepEntry(r, reqs[r][:-1], [len(reqs[r]) - 2]) for r in order]).cpu().numpy()
    b = eng.step([StepEntry(r, reqs[r][-1:], [0]) for r in order]).cpu().numpy()
    for i, r in enumerate(order):
        np.testing.assert_allclose(np.stack([a[i], b[i]]), alone[r], rtol=1e-5, atol=1e-5)


def _sharp(t):
    """Attention that all but picks one key, and a recurrent state that all but never forgets: with these a key far back
    that is lost, or a state that is dropped, changes the logits by far more than the tolerance."""
    for n in list(t):
        if n.endswith("mix.q"):
            t[n] *= 12.0
        if n.endswith("mix.w0"):
            t[n] = t[n] * 0.1 - 6.0
        if n.endswith("mix.a.b"):
            t[n] = t[n] * 0.1 - 3.0


def test_keys_far_back_at_page_borders_and_a_long_memory(tmp_path, dev):
    """Sharpened weights (`_sharp`): a prompt of several hundred tokens, cut at and beside page borders, then decoded
    token by token across more page borders; every position wanted."""
    from sllm_b200.engine import Engine, StepEntry, build_model
    config, page = CONFIG_B, 8
    d = make_model(tmp_path, config, edit=_sharp, seed=11)
    ids = _requests(config["vocab"], (330,), seed=12)["r0"]
    cfg, w = plain.load_model(d)
    full = plain.forward(ids, cfg, w)
    # the sharpening does what it is meant to: zeroing the first 200 cached tokens would move the last logits visibly
    cut = plain.forward(ids[200:], cfg, w)
    assert np.abs(cut[-1] - full[-1]).max() > 0.05
    want = {"r0": full.astype(np.float32)}
    for dtype in dtypes_on(dev):
        model, _ = build_model(d, dtype, dev)
        tr = traces.Trace()
        at = 0
        for n in (page - 1, 1, 1, page, 2 * page + 1, 64, 127, 2, 63):          # up to, onto and over page borders
            tr.step([("r0", at, ids[at:at + n], range(n))])
            at += n
        while at < len(ids):
            tr.step([("r0", at, ids[at:at + 1], [0])], end=["r0"] if at == len(ids) - 1 else [])
            at += 1
        eng = Engine(model, page_size=page, num_pages=tr.max_tokens // page, max_requests=1, poison_freed=True)
        out = traces.replay_engine(tr, eng)
        compare(tr, out, want, dtype, f"far/{dtype}")


def test_long_decoding_from_a_short_prompt(tmp_path, dev):
    """Three tokens of prompt, then 220 tokens one at a time: the recurrent state, the shift state and the latent cache carry
    everything, across many pages; every step's logits against the plain implementation."""
    from sllm_b200.engine import Engine, build_model
    d = make_model(tmp_path, CONFIG_A, seed=41)
    reqs = _requests(CONFIG_A["vocab"], (223,), seed=42)
    want = plain_logits(d, reqs)
    for dtype in dtypes_on(dev):
        model, _ = build_model(d, dtype, dev)
        tr = traces.tail_decode(reqs, tail=220)
        eng = Engine(model, page_size=8, num_pages=tr.max_tokens // 8, max_requests=1)
        compare(tr, traces.replay_engine(tr, eng), want, dtype, f"long/{dtype}")


def test_greedy_generation_through_the_entry_point(tmp_path, dev):
    """`LLM.generate`: admission, the token budget, prompts in portions, decoding (from captured graphs on the GPU),
    sampling on the device; against greedy decoding with the plain implementation."""
    from sllm_b200.engine import build_model
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    d = make_model(tmp_path, CONFIG_A, seed=21)
    cfg, w = plain.load_model(d)
    prompts = list(_requests(CONFIG_A["vocab"], (9, 40, 17, 3, 26), seed=22).values())
    new = 12
    model, _ = build_model(d, "float32", dev)
    llm = LLM(model=model, block_size=16, num_pages=40, max_num_seqs=3, chunk_size=16, max_batch_tokens=48, max_model_len=128)
    res = llm.generate(prompts, SamplingParams(max_new=new))
    for pr, r in zip(prompts, res):
        ids, out = list(pr), []
        for _ in range(new):
            logits = plain.forward(ids, cfg, w)[-1]
            top = np.sort(logits)[-2:]
            out.append(int(np.argmax(logits)))
            ids.append(out[-1])
            if top[1] - top[0] < 1e-3:      # a tie the rounding may break either way: compare up to here
                break
        assert r.ids[:len(out)] == out, (len(pr), r.ids, out)
    llm.engine.cache.check()
    assert not llm.engine.cache.requests


def test_command_line_with_random_weights(tmp_path, capsys, dev, monkeypatch):
    """The shipped recipe through ``python -m sllm_b200.serving.main``: plan mode describes the model's cache needs, run
    mode generates from a random model of the recipe's geometry."""
    import sllm_b200.engine.llm as llm_mod
    from sllm_b200.serving import main as cli
    recipe = "tiny-rososun"
    if dev == "cpu":
        import yaml
        real = llm_mod.LLM
        monkeypatch.setattr(llm_mod, "LLM", lambda model_dir, **kw: real(model_dir, **dict(kw, device="cpu")))
        with open(os.path.join(cli.RECIPES_DIR, "tiny-rososun.yaml")) as f:
            raw = yaml.safe_load(f)
        raw["memory"] = {"kv_device_bytes": 1 << 20}        # (without a device there is no free memory to ask for)
        recipe = os.path.join(str(tmp_path), "tiny-rososun.yaml")
        with open(recipe, "w") as f:
            yaml.safe_dump(raw, f)
    assert cli.main([recipe]) == 0
    out = capsys.readouterr().out
    assert "Rososun: 3 layers in 4 runs" in out and "latent vectors of 40" in out and "state slots: 4 runs" in out
    assert cli.main([recipe, "--mode", "run", "--random-weights", "4", "--prompt-ids", "5,17,3,150,42", "--max-new", "5",
                     "--dtype", "float32", "--log-level", "ERROR"]) == 0
    got = [int(t) for t in capsys.readouterr().out.strip().split(",")]
    assert len(got) == 5 and all(0 <= t < 320 for t in got)


@pytest.mark.gpu
def test_replay_program_on_a_model_folder(tmp_path):
    """bin/trace_run as a user runs it: the model class chosen by config.json, all four cuttings in one trace."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    d = make_model(tmp_path, CONFIG_B, seed=31)
    reqs = _requests(CONFIG_B["vocab"], (40, 75, 9), seed=32)
    want = traces.tagged(plain_logits(d, reqs))
    tr = traces.all_modes(reqs)
    for dtype in ("float32", "bfloat16"):
        out_dir = os.path.join(str(tmp_path), f"out_{dtype}")
        out = traces.replay_subprocess(tr, d, dtype, out_dir, 16)
        compare(tr, out, want, dtype, f"replay/{dtype}")
