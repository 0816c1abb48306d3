"""The Zuzunex decoder in the engine against the plain implementation (``plain_zuzunex``).

Every test that needs a kernel set takes the fixture ``kit``: the plain tensor-op set on the CPU
(``ref_kernels.RefKernels``, which checks the engine's bookkeeping: cache, state slots, batching, scheduling), and
under ``-m gpu`` the CUDA sets in float32 and bfloat16.  Configurations are made here, with random weights; they
differ from one another in every size.
"""

from __future__ import annotations

import copy
import math

import pytest
import torch

import helpers
import plain_zuzunex as pz
from ref_kernels import RefKernels

from distie_b200.cache.manager import pages_needed
from distie_b200.config import ConfigError, EngineConfig, ZuzunexConfig, get_architecture
from distie_b200.engine.batch import BatchEntry, lay_out, views
from distie_b200.engine.engine import Engine, GenerateRequest
from distie_b200.engine.trace_replay import TraceSession
from distie_b200.kernels.interface import KvSlot, RotaryTable
from distie_b200.models.decoder import model_tensor_specs
from distie_b200.parts.position import ramped_frequencies


def _plain(heads, kv_heads, dim, vdim, scale, cap=None, temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if cap is not None:
        m["softcap"] = cap
    if temp is not None:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return m


def _conv(heads, kv_heads, dim, vdim, scale, taps=None, rot=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if taps is not None:
        m["conv"] = taps
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, identity, top, ff, shared):
    return {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": ff},
            "shared": None if shared is None else {"ff": shared}}


# Small: every branch once.  The first two layers run three times; values of another size than keys; a temperature
# that steps every five positions; a ramp that slows half of the rotated pairs.
SMALL = {
    "architecture": "Zuzunex", "vocab": 96, "width": 48, "norm": {"eps": 1e-5}, "logit_scale": 1.5,
    "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        _layer("attention_2", _conv(4, 2, 12, 8, 0.3, 4, (1000.0, 8), (3.0, 16, 4.0, 1.0)), _moe(5, 2, 3, 16, 24)),
        _layer("attention", _plain(3, 3, 8, 10, 0.5, 5.0, (0.7, 5)), _dense(40)),
        _layer("attention", _plain(2, 1, 16, 16, 0.25), None),
    ],
}
# Awkward: no loop; a loop of one pass would be the same.  A single head and five; sizes that are no powers of two;
# a convolution of two taps and none; whole heads rotated without scaling; no rotation at all; as many chosen experts
# as router outputs; no identity experts; no shared expert; one expert chosen; a logit scale left out; pages of four.
AWKWARD = {
    "architecture": "Zuzunex", "vocab": 101, "width": 72, "norm": {"eps": 1e-6},
    "layers": [
        _layer("attention", _plain(1, 1, 24, 10, 0.2, None, (1.3, 1)), _moe(3, 1, 4, 20, None)),
        _layer("attention_2", _conv(5, 5, 6, 14, 0.4, 2, (10.0, 6)), _moe(4, 0, 1, 16, 8)),
        _layer("attention_2", _conv(6, 2, 10, 3, 0.3, None, None), _dense(50)),
        _layer("attention", _plain(4, 2, 14, 6, 0.3, 0.8, None), _moe(2, 3, 2, 12, 24)),
        _layer("attention_2", _conv(2, 1, 20, 20, 0.22, 5, (1e6, 4), (8.0, 8, 2.0, 0.5)), None),
    ],
}
# Sizes of a real model's order: head sizes 64 and 128 (in bfloat16 the tensor-core attention kernels and, in steps
# of more than 128 tokens, the tensor-core products run); the middle layers run twice.
WIDE = {
    "architecture": "Zuzunex", "vocab": 500, "width": 256, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        _layer("attention", _plain(4, 2, 64, 64, 0.125, 20.0, (0.5, 32)), _dense(384)),
        _layer("attention_2", _conv(4, 1, 128, 128, 0.09, 3, (10000.0, 64), (4.0, 64, 8.0, 1.0)), _moe(8, 1, 2, 64, 128)),
        _layer("attention_2", _conv(6, 3, 80, 48, 0.11, 2, (10000.0, 80)), _moe(4, 0, 2, 32, None)),
        _layer("attention", _plain(16, 1, 64, 64, 0.13, None, None), None),
    ],
}
CONFIGS = {"small": (SMALL, 4, 0), "awkward": (AWKWARD, 4, 1), "wide": (WIDE, 16, 2)}

FP32_TOL = 1e-4    # rms over the vocabulary of the logits' difference, mean taken off, over the logit scale
BF16_TOL = 6e-2

KITS = ["cpu", pytest.param("gpu32", marks=pytest.mark.gpu), pytest.param("gpu16", marks=pytest.mark.gpu)]
ORACLE = {"stored": None}  # the type whose roundings the plain implementation takes on for the kit in use


@pytest.fixture(params=KITS)
def kit(request):
    ORACLE["stored"] = torch.bfloat16 if request.param == "gpu16" else None
    if request.param == "cpu":
        return RefKernels(torch.float32, "cpu")
    from distie_b200.kernels import make_kernels

    return make_kernels(torch.float32 if request.param == "gpu32" else torch.bfloat16, "cuda:0")


def tolerance(kit) -> float:
    return FP32_TOL if kit.dtype == torch.float32 else BF16_TOL


def every_expert(cfg: dict) -> dict:
    """``cfg`` with every router choosing all of its outputs: the weights still vary with the token, but no choice
    can be turned around by rounding."""
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            router = layer["mlp"]["router"]
            router["top"] = router["experts"] + router.get("identity", 0)
    return out


def model(name: str, kit=None):
    """The configuration, its page size and random weights.  For the bfloat16 engine the routers choose every output
    (a choice that hangs on less than 16-bit activations can tell apart changes the token's keys in every later
    layer); the float32 engines run the choices everywhere, and ``test_clear_choices_in_sixteen_bits`` runs them in
    bfloat16 where they are clear."""
    cfg, page, seed = CONFIGS[name]
    cfg = every_expert(cfg) if kit is not None and kit.dtype != torch.float32 else copy.deepcopy(cfg)
    return cfg, page, pz.random_weights(cfg, seed)


def engine_of(cfg, weights, page, kit, num_blocks: int, max_seqs: int = 4, **knobs):
    arch = get_architecture(cfg["architecture"])
    dtype = "float32" if kit.dtype == torch.float32 else "bfloat16"
    config = EngineConfig(num_blocks=num_blocks, page_size=page, max_seqs=max_seqs, dtype=dtype, device=str(kit.device),
                          decode_graphs=kit.device.type == "cuda", **{"token_budget": 4096, **knobs})
    stored = {k: v.to(torch.bfloat16) for k, v in weights.items()}
    return Engine.assemble(arch, arch.config_cls.from_dict(cfg), stored, kit, config)


def engine_for(name: str, kit, num_blocks: int, max_seqs: int = 4, **knobs):
    cfg, page, weights = model(name, kit)
    return engine_of(cfg, weights, page, kit, num_blocks, max_seqs, **knobs), cfg, weights


def plain_logits(cfg, weights, ids, margins=None) -> torch.Tensor:
    """The oracle: the plain implementation in float64; for the bfloat16 engine with that type's roundings where an
    engine stores 16 bits between two products (and nowhere else)."""
    with pz.stored_as(ORACLE["stored"]):
        return pz.forward(ids, weights, cfg, torch.float64, margins=margins).float()


def row_errors(have: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    diff = have.double() - want.double()
    diff = diff - diff.mean(-1, keepdim=True)
    return diff.pow(2).mean(-1).sqrt() / float(want.double().std())


def assert_close(got: dict, expected: dict, tol: float, what: str) -> None:
    expected = helpers.expected_for(got, expected)
    for rid, want in expected.items():
        errors = row_errors(got[rid], want)
        at = int(errors.argmax())
        assert float(errors[at]) <= tol, f"{what}: request {rid}, position {at}: {float(errors[at]):.3e} of the logit scale"


def requests_of(cfg, lengths, seed=20):
    return {f"r{i}": helpers.random_ids(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


def step_for(kit, entries):
    layout = lay_out([BatchEntry(*e) for e in entries])
    return views(torch.from_numpy(layout.packed).to(kit.device), layout)[0], layout


def in_slices(x: torch.Tensor) -> torch.Tensor:
    """``x`` as three slices ``[3, T, n]`` whose sum it is exactly, as a split product leaves it."""
    return torch.stack([x * 0.5, x * 0.25, x * 0.25])


def _close(have, want, tol, what):
    scale = float(want.double().abs().max()) or 1.0
    err = float((have.double().cpu() - want.double()).abs().max()) / scale
    assert err <= tol, f"{what}: {err:.3e} of the largest value"


# -- configuration and weights -----------------------------------------------------------------------------
def test_config_reads_every_size_and_names_what_is_missing():
    cfg = ZuzunexConfig.from_dict(AWKWARD)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.logit_scale, len(cfg.layers), cfg.loop) == (101, 72, 1e-6, 1.0, 5, None)
    first = cfg.layers[0].mixer
    assert (first.heads, first.kv_heads, first.dim, first.vdim, first.scale) == (1, 1, 24, 10, 0.2)
    assert (first.softcap, first.temp_coef, first.temp_every, first.biases, first.conv, first.rot_dims) == (None, 1.3, 1.0, False, None, None)
    last = cfg.layers[4].mixer
    assert (last.conv, last.rot_base, last.rot_dims, last.biases, last.weighted_norm) == (5, 1e6, 4, True, True)
    assert (last.rot_scaling.factor, last.rot_scaling.original, last.rot_scaling.fast, last.rot_scaling.slow) == (8.0, 8.0, 2.0, 0.5)
    assert cfg.layers[2].mixer.conv is None and cfg.layers[2].mixer.rot_dims is None and cfg.layers[1].mixer.rot_scaling is None
    routed = cfg.layers[3].mlp
    assert (routed.experts, routed.identity, routed.top, routed.ff, routed.shared_ff) == (2, 3, 2, 12, 24)
    assert cfg.layers[0].mlp.shared_ff is None and cfg.layers[2].mlp.ff == 50 and cfg.layers[4].mlp is None
    assert cfg.run_order() == [0, 1, 2, 3, 4]
    small = ZuzunexConfig.from_dict(SMALL)
    assert small.loop == (0, 2, 3) and small.run_order() == [0, 1, 0, 1, 0, 1, 2] and small.logit_scale == 1.5
    assert ZuzunexConfig.from_dict(WIDE).run_order() == [0, 1, 2, 1, 2, 3]
    spec = get_architecture("Zuzunex").recipe(small)
    assert [(c.layer, c.cache_slot, c.writes_cache) for c in spec.order] == [(l, s, True) for s, l in enumerate([0, 1, 0, 1, 0, 1, 2])]
    for path, match in (
        (("layers", 1, "mixer", "kv_heads"), r"layers\[1\]\.mixer\.kv_heads"),
        (("layers", 0, "mixer", "rot", "base"), r"layers\[0\]\.mixer\.rot\.base"),
        (("layers", 0, "mixer", "rot", "scaling", "slow"), r"layers\[0\]\.mixer\.rot\.scaling\.slow"),
        (("layers", 1, "mixer", "q_temp", "every"), r"layers\[1\]\.mixer\.q_temp\.every"),
        (("layers", 0, "mlp", "router", "top"), r"layers\[0\]\.mlp\.router\.top"),
        (("layers", 0, "mlp", "expert"), r"layers\[0\]\.mlp\.expert"),
        (("loop", "times"), r"loop\.times"),
        (("norm",), "norm"),
        (("width",), "width"),
    ):
        broken = copy.deepcopy(SMALL)
        at = broken
        for key in path[:-1]:
            at = at[key]
        del at[path[-1]]
        with pytest.raises(ConfigError, match=match):
            ZuzunexConfig.from_dict(broken)
    for change, match in (
        (lambda c: c["layers"][0].update(type="latent_attention"), "latent_attention"),
        (lambda c: c["layers"][1]["mlp"].update(kind="swiglu"), "swiglu"),
        (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
        (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14), "dims"),
        (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "top"),
        (lambda c: c["loop"].update(stop=4), "loop"),
        (lambda c: c["loop"].update(times=0), "loop"),
    ):
        broken = copy.deepcopy(SMALL)
        change(broken)
        with pytest.raises(ConfigError, match=match):
            ZuzunexConfig.from_dict(broken)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    cfg = CONFIGS[name][0]
    arch = get_architecture("Zuzunex")
    declared = {s.name: tuple(s.shape) for s in model_tensor_specs(arch.recipe(arch.config_cls.from_dict(cfg)))}
    assert declared == {k: tuple(v) for k, v in pz.tensor_shapes(cfg).items()}


def test_random_model_folder_loads_by_its_config(tmp_path):
    from distie_b200.config import read_config
    from distie_b200.weights import write_random_model

    folder = write_random_model(str(tmp_path / "m"), SMALL, seed=3, std=0.1, norm_noise=0.05)
    arch, cfg = read_config(folder)
    assert arch.name == "Zuzunex" and cfg.width == 48
    engine = Engine.assemble(arch, cfg, folder, RefKernels(torch.float32),
                             EngineConfig(num_blocks=8, page_size=16, max_seqs=2, dtype="float32", device="cpu", decode_graphs=False))
    # every pass of a layer that runs again has a cache slot (and, where it convolves, a state slot) of its own
    assert engine.model.spec.num_cache_slots == 7 and len(engine.model.blocks) == 3
    out = engine.generate([[1, 2, 3]], max_new_tokens=3, ignore_eos=True)
    assert len(out[0].token_ids) == 3


def test_frequencies_slowed_along_a_ramp():
    for base, dims, scaling in ((1000.0, 8, (3.0, 16, 4.0, 1.0)), (10000.0, 64, (4.0, 64, 8.0, 1.0)), (1e6, 4, (8.0, 8, 2.0, 0.5)),
                                (2e5, 40, (5.0, 2048, 16.0, 2.0)), (100.0, 16, (2.0, 4096, 1.0, 1.0))):
        want, mult = pz.yarn_frequencies(base, dims, dict(zip(("factor", "original", "fast", "slow"), scaling)))
        got = ramped_frequencies(base, dims, *scaling)
        assert torch.allclose(got.double(), want, rtol=1e-6, atol=0)
        assert mult == pytest.approx(0.1 * math.log(scaling[0]) + 1.0)
    plain, one = pz.yarn_frequencies(100.0, 6, None)
    assert one == 1.0 and torch.allclose(plain, 100.0 ** (-torch.arange(3, dtype=torch.float64) / 3))


# -- each mechanism alone: ops of the kernel set against the plain functions ------------------------------------
def _slot(kit, kv_heads, dim, vdim, pages, page_size, table):
    dev = kit.device
    k = torch.zeros(pages, kv_heads, page_size, dim, dtype=kit.dtype, device=dev)
    v = torch.zeros(pages, kv_heads, page_size, vdim, dtype=kit.dtype, device=dev)
    return KvSlot(k, v, torch.tensor(table, dtype=torch.int32, device=dev), page_size, pages)


def _cached(kv, seat, positions, values=False):
    dev = kv.k.device
    pages = kv.block_table[seat, (positions // kv.page_size).to(dev)].long()
    return (kv.v if values else kv.k)[pages, :, (positions % kv.page_size).to(dev)]


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot,scaling,weights,temp,page", [
    (4, 2, 12, 8, 8, (3.0, 16, 4.0, 1.0), True, None, 4),
    (3, 3, 8, 10, 0, None, False, (0.7, 5), 4),
    (1, 1, 24, 24, 24, None, True, (1.3, 1), 8),
    (4, 1, 128, 128, 64, (4.0, 64, 8.0, 1.0), True, None, 16),
    (8, 4, 64, 64, 0, None, False, (0.5, 32), 16),
    (6, 3, 80, 48, 80, None, True, None, 16),
    (2, 2, 40, 7, 6, (8.0, 8, 2.0, 0.5), False, (0.25, 3), 4),
])
def test_projection_normed_rotated_tempered_and_stored(kit, heads, kv_heads, dim, vdim, rot, scaling, weights, temp, page):
    """From the float32 projection (whole, and as slices with a bias; more columns behind q, k and v are not read)
    to q and the pages, which are handed out in reverse: the norm comes before the rotation, its weight is shared by
    the heads, the temperature multiplies q only and steps where ``floor((p + 1) / every)`` does, values have a size
    of their own."""
    g = torch.Generator().manual_seed(dim + vdim + heads)
    n, first, eps = 45, 3, 1e-5
    columns = (heads + kv_heads) * dim + kv_heads * vdim
    proj = torch.randn(n, columns + 5, generator=g) * 2.0
    bias = torch.randn(columns, generator=g) * 0.3
    q_w = (1.0 + 0.3 * torch.randn(dim, generator=g)) if weights else None
    k_w = (1.0 + 0.3 * torch.randn(dim, generator=g)) if weights else None
    positions = torch.arange(first, first + n)
    table = None
    if rot:
        freq = ramped_frequencies(1000.0, rot, *scaling) if scaling else 1000.0 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot).float()
        table = RotaryTable(freq.to(kit.device), rot, False, 0.1 * math.log(scaling[0]) + 1.0 if scaling else 1.0)
    # the plain functions
    dense = (proj[:, :columns] + bias).double()
    q = dense[:, : heads * dim].view(n, heads, dim)
    k = dense[:, heads * dim : (heads + kv_heads) * dim].view(n, kv_heads, dim)
    v = dense[:, (heads + kv_heads) * dim :].view(n, kv_heads, vdim)
    q, k = pz.rms_unit(q, eps), pz.rms_unit(k, eps)
    if weights:
        q, k = q * q_w.double(), k * k_w.double()
    if rot:
        f, mult = pz.yarn_frequencies(1000.0, rot, dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None)
        q, k = pz.rotate_half(q, positions, f, mult, rot), pz.rotate_half(k, positions, f, mult, rot)
    if temp:
        q = q * pz.query_temperature(positions, temp[0], temp[1], torch.float64)[:, None, None]
    dev = kit.device
    width = pages_needed(first + n, page)
    for source, b in ((in_slices(proj), bias), (proj + torch.cat([bias, torch.zeros(5)]), None)):
        kv = _slot(kit, kv_heads, dim, vdim, width + 1, page, [[-1] * width, list(range(width - 1, -1, -1))])
        step, _ = step_for(kit, [(1, [0] * n, first, ())])
        q_out = torch.empty(n, heads * dim, dtype=kit.dtype, device=dev)
        kit.qkv_norm_write(source.to(dev), b.to(dev) if b is not None else None, step, kv, table, heads, kv_heads, dim, vdim, eps,
                           q_w.to(dev) if weights else None, k_w.to(dev) if weights else None, temp, q_out)
        if hasattr(kit, "check_errors"):
            kit.check_errors()
        tol = 2e-5 if kit.dtype == torch.float32 else 1e-2
        _close(q_out.float().view(n, heads, dim), q, tol, "q")
        _close(_cached(kv, 1, positions).float(), k, tol, "k in its pages")
        _close(_cached(kv, 1, positions, values=True).float(), v, tol, "v in its pages")
    # without a cache slot only q is made (a call that reads another call's pages)
    q_only = torch.empty(n, heads * dim, dtype=kit.dtype, device=dev)
    kit.qkv_norm_write(source.to(dev), None, step, None, table, heads, kv_heads, dim, vdim, eps,
                       q_w.to(dev) if weights else None, k_w.to(dev) if weights else None, temp, q_only)
    assert torch.equal(q_only, q_out)


def _plain_attention(q, k, v, scale, sink, cap):
    return pz.sink_attention(q, k, v, scale, sink, cap)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,page,n,cap", [
    (3, 3, 8, 10, 4, 61, 5.0), (4, 2, 12, 8, 4, 90, None), (4, 2, 64, 64, 16, 300, 20.0), (4, 1, 128, 128, 16, 200, None),
    (16, 1, 64, 64, 32, 270, 3.0), (8, 8, 128, 128, 8, 150, 30.0), (6, 3, 80, 48, 16, 140, None), (2, 1, 32, 32, 4, 75, 1.5),
    (5, 5, 16, 16, 8, 130, None), (12, 2, 64, 64, 24, 190, 8.0),
])
def test_capped_scores_and_a_sink_with_keys_that_stand_out(kit, heads, kv_heads, dim, vdim, page, n, cap):
    """Keys and values go through pages handed out in reverse; attention runs in portions and token by token.  Every
    query looks for one direction; the very first key, the keys on either side of every fourth page border and every
    seventh key carry it with a strength of their own, so one far key among hundreds decides most of an output, and
    with a cap the strongest ones are levelled.  Head 0's sink is far above every score (its output all but
    vanishes), the last head's far below (a plain softmax), the others' lie among the scores."""
    g = torch.Generator().manual_seed(dim + vdim + n)
    q = torch.randn(n, heads, dim, generator=g) * 0.3
    k = torch.randn(n, kv_heads, dim, generator=g) * 0.5
    v = torch.randn(n, kv_heads, vdim, generator=g)
    a = torch.randn(dim, generator=g)
    a = a / a.norm()
    q = q + 3.0 * a
    marked = {0: 6.0}
    for border in range(4 * page, n, 4 * page):
        marked[border - 1], marked[border] = 4.0 + (border % 3), 5.5 - (border % 2)
    for j in range(3, n, 7):
        marked.setdefault(j, 2.0 + (j * 5 % 9) * 0.4)
    for j, strength in marked.items():
        k[j] = strength * a + 0.1 * torch.randn(kv_heads, dim, generator=g)
    sink = torch.randn(heads, generator=g) * 3 + 6
    sink[0] = 60.0
    sink[-1] = -60.0
    if kit.dtype != torch.float32:
        q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    scale = 0.8
    want = _plain_attention(q.double(), k.double(), v.double(), scale, sink.double(), cap)
    dev = kit.device
    width = pages_needed(n, page)
    table = [[-1] * width, list(range(width - 1, -1, -1))]
    tol = 2e-5 if kit.dtype == torch.float32 else 3e-2
    for cuts in ([1, 1, 2, page - 1, 1, 1, 2, 3 * page, 1, 1, 1, 4 * page + 1, 2], [n]):
        kv = _slot(kit, kv_heads, dim, vdim, width + 1, page, table)
        got, at = [], 0
        cuts = list(cuts)
        while at < n:
            count = min(cuts.pop(0) if cuts else 1, n - at)
            step, _ = step_for(kit, [(1, [0] * count, at, ())])
            rows = torch.arange(at, at + count)
            pages = kv.block_table[1, (rows // page).to(dev)].long()
            kv.k[pages, :, (rows % page).to(dev)] = k[at : at + count].to(dev, kit.dtype)
            kv.v[pages, :, (rows % page).to(dev)] = v[at : at + count].to(dev, kit.dtype)
            out = torch.empty(count, heads * vdim, dtype=kit.dtype, device=dev)
            kit.attention(q[at : at + count].reshape(count, -1).contiguous().to(dev, kit.dtype), out, step, kv, heads, kv_heads, dim,
                          None, scale, None, 0, cap or 0.0, sink.to(dev))
            got.append(out.float().cpu())
            at += count
        if hasattr(kit, "check_errors"):
            kit.check_errors()
        have = torch.cat(got).view(n, heads, vdim)
        _close(have, want, tol, "attention with a sink")
        if heads > 1:  # the sink took all of head 0's weight
            assert float(have[:, 0].abs().max()) < 1e-6 * float(want.abs().max()) + 1e-12
    # without a sink and without a cap: the plain softmax of the same kernels
    kit.attention(q[at - count : at].reshape(count, -1).contiguous().to(dev, kit.dtype), out, step, kv, heads, kv_heads, dim, None, scale)
    plain = _plain_attention(q.double(), k.double(), v.double(), scale, torch.full((heads,), -1e30, dtype=torch.float64), None)
    _close(out.float().view(count, heads, vdim), plain[at - count : at], tol, "no sink, no cap")
    if kit.device.type == "cuda" and kit.dtype == torch.bfloat16 and dim == vdim and dim in (64, 128):
        ran = kit.kernel_counts
        assert ran.get("attention_decode_mma") and (ran.get("attention_prefill_tcgen05") or ran.get("attention_prefill"))
        assert not ran.get("attention_generic")


@pytest.mark.parametrize("channels,taps,extra", [(36, 4, 12), (40, 2, 0), (52, 5, 3), (1024, 3, 512), (9, 1, 0), (64, 4, 64)])
def test_convolution_behind_a_biased_projection(kit, channels, taps, extra):
    """Two requests in one step and then in portions of several sizes, down to single tokens: the bias joins every
    input of the step, a request's first tokens see zeros (not the bias) before its start, and the state slot of a
    seat carries the last ``taps - 1`` biased inputs from one step to the next."""
    g = torch.Generator().manual_seed(channels + taps)
    lengths = {2: 23, 1: 9}
    x = {seat: torch.randn(n, channels + extra, generator=g) for seat, n in lengths.items()}
    bias = torch.randn(channels, generator=g)
    weight = torch.randn(channels, taps, generator=g)
    want = {seat: pz.causal_conv((x[seat][:, :channels] + bias).double(), weight.double()) for seat in x}
    dev = kit.device
    for portions in ({2: [23], 1: [9]}, {2: [1, 2, 1, 7, 1, 1, 10], 1: [2, 1, 1, 5]}):
        state = torch.zeros(3, max(taps - 1, 0), channels, dtype=torch.float32, device=dev) if taps > 1 else None
        done = {seat: 0 for seat in x}
        got = {seat: [] for seat in x}
        portions = {seat: list(p) for seat, p in portions.items()}
        while any(portions.values()):
            entries, order = [], []
            for seat in sorted(portions, key=lambda s: (portions[s][0] if portions[s] else 0) != 1):  # single tokens first
                if portions[seat]:
                    count = portions[seat].pop(0)
                    entries.append((seat, [0] * count, done[seat], ()))
                    order.append((seat, count))
            step, layout = step_for(kit, entries)
            rows = torch.cat([x[seat][done[seat] : done[seat] + count] for seat, count in order])
            out = kit.short_conv(in_slices(rows).to(dev)[..., :channels], weight.to(dev), None, state, step, "none",
                                 input_bias=bias.to(dev))
            at = 0
            for seat, count in order:
                got[seat].append(out[at : at + count].cpu())
                at += count
                done[seat] += count
        for seat in x:
            _close(torch.cat(got[seat]), want[seat], 2e-5, f"convolution, seat {seat}")


@pytest.mark.parametrize("experts,identity,top,width", [(5, 2, 3, 48), (3, 1, 4, 72), (4, 0, 1, 40), (2, 3, 2, 64), (8, 1, 2, 256), (16, 0, 4, 128)])
def test_softmax_scores_a_correction_for_the_choice_and_renormalised_weights(kit, experts, identity, top, width):
    g = torch.Generator().manual_seed(experts * 7 + top)
    outputs = experts + identity
    for tokens in (9, 150):
        x = torch.randn(tokens, width, generator=g)
        router = torch.randn(outputs, width, generator=g) * 3.0 / math.sqrt(width)
        correction = torch.randn(outputs, generator=g) * 0.3
        if kit.dtype != torch.float32:
            x, router = (t.to(torch.bfloat16).float() for t in (x, router))
        scores = torch.softmax(x.double() @ router.double().T, -1)
        chosen = pz.choose_experts(scores, correction.double(), top)
        dev = kit.device
        ids, weights = kit.route_top(x.to(dev, kit.dtype), router.to(dev, kit.dtype), top, "softmax", None, 1.0, 0, correction.to(dev), True)
        clear = pz.choice_margin(scores, correction.double(), top) > (1e-5 if kit.dtype == torch.float32 else 2e-3)
        assert int(clear.sum()) >= tokens // 2
        for t in range(tokens):
            if not bool(clear[t]):
                continue
            assert sorted(ids[t].tolist()) == sorted(chosen[t]), f"token {t}"
            picked = scores[t, ids[t].long().cpu()]
            _close(weights[t], picked / (picked.sum() + 1e-20), 1e-5 if kit.dtype == torch.float32 else 2e-2, "weights")
        # the correction changes choices and never weights: with a large one on the last output it is always chosen
        push = torch.zeros(outputs)
        push[-1] = 10.0
        ids2, weights2 = kit.route_top(x.to(dev, kit.dtype), router.to(dev, kit.dtype), top, "softmax", None, 1.0, 0, push.to(dev), True)
        assert bool((ids2 == outputs - 1).any(-1).all()) and float((weights2.sum(-1) - 1).abs().max()) < 1e-5


@pytest.mark.parametrize("experts,identity,top,width,ff,tokens", [(5, 2, 3, 48, 16, 9), (3, 1, 4, 72, 20, 40), (2, 3, 2, 64, 12, 7),
                                                                  (8, 1, 2, 256, 64, 300), (4, 0, 2, 128, 32, 70)])
def test_experts_that_return_their_input_among_gated_experts(kit, experts, identity, top, width, ff, tokens):
    g = torch.Generator().manual_seed(experts + identity + tokens)
    x = torch.randn(tokens, width, generator=g)
    w = {}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"] = (torch.randn(ff, width, generator=g) / math.sqrt(width) for _ in range(2))
        w[f"e{e}.down"] = torch.randn(width, ff, generator=g) / math.sqrt(ff)
    ids = torch.stack([torch.randperm(experts + identity, generator=g)[:top] for _ in range(tokens)]).to(torch.int32)
    if identity:
        ids[0] = torch.arange(experts + identity - top, experts + identity)[:top] if top <= identity else ids[0]
    weights = torch.rand(tokens, top, generator=g)
    if kit.dtype != torch.float32:
        x = x.to(torch.bfloat16).float()
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    wd = {k: v.double() for k, v in w.items()}
    want = torch.zeros(tokens, width, dtype=torch.float64)
    with pz.stored_as(None if kit.dtype == torch.float32 else torch.bfloat16):
        for t in range(tokens):
            for e, s in zip(ids[t].tolist(), weights[t].double()):
                want[t] += s * (x[t].double() if e >= experts else pz.gated_ff(x[t : t + 1].double(), wd, f"e{e}.")[0])
    dev = kit.device
    gate_up = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(experts)]).to(dev, kit.dtype)
    down = torch.stack([w[f"e{e}.down"] for e in range(experts)]).to(dev, kit.dtype)
    out = kit.routed_swiglu(x.to(dev, kit.dtype), ids.to(dev), weights.to(dev), gate_up, down, False, None, identity)
    assert out.shape == (top, tokens, width) and out.dtype == torch.float32
    _close(out.sum(0), want, 2e-5 if kit.dtype == torch.float32 else 2e-2, "experts and identity experts")
    if hasattr(kit, "check_errors"):
        kit.check_errors()


@pytest.mark.parametrize("tokens,columns", [(5, 48), (70, 30), (130, 512)])
def test_gate_element_by_element(kit, tokens, columns):
    g = torch.Generator().manual_seed(columns)
    x = torch.randn(tokens, columns, generator=g)
    logits = torch.randn(tokens, columns + 8, generator=g) * 2
    if kit.dtype != torch.float32:
        x = x.to(torch.bfloat16).float()
    dev = kit.device
    have = x.to(dev, kit.dtype).clone()
    kit.head_gate(have, in_slices(logits).to(dev)[..., 8:] if columns % 4 == 0 else in_slices(logits).to(dev)[..., 3 : 3 + columns], columns)
    want = x.double() * torch.sigmoid((logits[:, 8:] if columns % 4 == 0 else logits[:, 3 : 3 + columns]).double())
    _close(have.float(), want, 1e-5 if kit.dtype == torch.float32 else 1e-2, "gate")


# -- each kind of layer alone in a model, then all of them ---------------------------------------------------
ALONE = {
    "capped": [_layer("attention", _plain(3, 1, 8, 6, 0.6, 2.0, (0.9, 4)), None)],
    "bare": [_layer("attention", _plain(2, 2, 16, 16, 0.3), None)],
    "convolved": [_layer("attention_2", _conv(4, 2, 8, 8, 0.4, 3, (300.0, 6), (2.0, 8, 2.0, 1.0)), None)],
    "biased": [_layer("attention_2", _conv(2, 1, 12, 5, 0.4), None)],
    "one_tap": [_layer("attention_2", _conv(3, 1, 8, 8, 0.4, 1, (100.0, 2)), None)],
    "odd_steps": [_layer("attention", _plain(2, 2, 8, 8, 0.5, 4.0, (0.6, 2.5)), None)],
    "dense": [_layer("attention", _plain(1, 1, 8, 8, 0.3), _dense(44))],
    "routed": [_layer("attention", _plain(1, 1, 8, 8, 0.3), _moe(6, 2, 3, 20, 28))],
    "again": [_layer("attention_2", _conv(2, 2, 8, 8, 0.4, 4, (50.0, 8)), _dense(24))],
}


@pytest.mark.parametrize("kind", list(ALONE))
def test_one_layer_of_a_kind_prefill_against_single_tokens(kit, kind):
    cfg = {"architecture": "Zuzunex", "vocab": 60, "width": 56, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
           "layers": copy.deepcopy(ALONE[kind])}
    if kind == "again":
        cfg["loop"] = {"start": 0, "stop": 1, "times": 4}
    if kit.dtype != torch.float32:
        cfg = every_expert(cfg)
    weights = pz.random_weights(cfg, 40)
    requests = requests_of(cfg, [41, 6], seed=70)
    expected = {rid: plain_logits(cfg, weights, ids) for rid, ids in requests.items()}
    for schedule in (helpers.schedule_whole, lambda r: helpers.schedule_tail(r, tail=25)):
        steps = schedule(requests)
        engine = engine_of(cfg, weights, 4, kit, num_blocks=pages_needed(41, 4) + 2, max_seqs=2)
        got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
        assert_close(got, expected, tolerance(kit), kind)


@pytest.mark.gpu
def test_clear_choices_in_sixteen_bits():
    """The bfloat16 engine with routers that choose a few of their outputs, on prompts whose every choice is clear
    (found by trying seeds against the plain implementation): whole prompts, prefill against single tokens,
    portions."""
    from distie_b200.kernels import make_kernels

    kit = make_kernels(torch.bfloat16, "cuda:0")
    ORACLE["stored"] = torch.bfloat16
    cfg, page, weights = copy.deepcopy(SMALL), 4, pz.random_weights(SMALL, 0, router_gain=10.0)
    requests = {}
    for seed in range(400, 2400):
        ids = helpers.random_ids(cfg["vocab"], 7, seed)
        margins = []
        plain_logits(cfg, weights, ids, margins)
        if float(torch.stack(margins).min()) >= 0.06:  # of the last chosen score
            requests[f"c{len(requests)}"] = ids
            if len(requests) == 3:
                break
    assert len(requests) == 3, "no prompts with clear choices among the seeds tried"
    expected = {rid: plain_logits(cfg, weights, ids) for rid, ids in requests.items()}
    for schedule in (helpers.schedule_whole, lambda r: helpers.schedule_tail(r, tail=5), helpers.schedule_portions):
        steps = schedule(requests)
        engine = engine_of(cfg, weights, page, kit, num_blocks=16, max_seqs=2)
        got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
        assert_close(got, expected, BF16_TOL, "clear choices")
    assert kit.kernel_counts.get("routed_swiglu") and kit.kernel_counts.get("route_top")


LENGTHS = {"small": [70, 1, 29, 51], "awkward": [45, 3, 23, 38], "wide": [230, 97, 2, 140]}
SCHEDULES = {
    "whole": helpers.schedule_whole,
    "tail": lambda r: helpers.schedule_tail(r, tail=30),
    "portions": helpers.schedule_portions,
    "mixed": lambda r: helpers.schedule_mixed(r, seed=5, live_max=3, refeed=1),
}


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("mode", list(SCHEDULES))
def test_replay_against_plain(kit, name, mode):
    """Whole prompts, prefill against token-by-token decoding, portions down to two tokens, and batches of unequal
    requests (portions beside single tokens, a request given up and fed again) in a pool made for the schedule's
    peak and three seats, so that pages, seats and state slots are used again."""
    if name == "wide" and kit.device.type == "cpu" and mode != "mixed":
        pytest.skip("the wide configuration runs on the CPU in one mode only: it is slow there")
    cfg, page, weights = model(name, kit)
    requests = requests_of(cfg, LENGTHS[name])
    steps = SCHEDULES[mode](requests)
    peak = helpers.peak_tokens(steps, granule=page)
    engine, _, _ = engine_for(name, kit, num_blocks=pages_needed(peak, page), max_seqs=3)
    got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
    expected = {rid: plain_logits(cfg, weights, ids) for rid, ids in requests.items()}
    assert_close(got, expected, tolerance(kit), f"{name}/{mode}")
    assert engine.cache.free_seats == 3 and all(g.pool.num_free == g.num_pages for g in engine.cache.groups)
    if kit.device.type == "cuda":
        ran = kit.kernel_counts
        assert ran.get("qkv_norm_write") and ran.get("head_gate") and ran.get("routed_swiglu") and ran.get("add_layernorm")
        if name == "wide" and kit.dtype == torch.bfloat16:
            assert ran.get("attention_prefill_tcgen05") and (mode in ("whole", "portions") or ran.get("attention_decode_mma"))


@pytest.mark.parametrize("name", ["small", "awkward"])
def test_cuts_at_around_and_across_page_borders(kit, name):
    """The first tokens one by one; portions that end just before, at and just after page borders; two tokens at a
    time across one; then single tokens across the next ones (and, for the temperature of ``small``, across the
    positions where its step function moves on)."""
    cfg, page, weights = model(name, kit)
    ids = helpers.random_ids(cfg["vocab"], 6 * page + 5, 77)
    cuts = [1, 1, 1, page - 4 if page > 4 else 1, 2, page - 1, 1, 1, page, 2, 2, page + 1, 1, 1, 2 * page - 3, 2]
    steps, at = [], 0
    while at < len(ids):
        size = min(max(1, cuts.pop(0)) if cuts else 1, len(ids) - at)
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": ids[at : at + size], "want": list(range(size))}],
                      "end": ["a"] if at + size == len(ids) else []})
        at += size
    engine, _, _ = engine_for(name, kit, num_blocks=pages_needed(len(ids), page))
    got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
    assert_close(got, {"a": plain_logits(cfg, weights, ids)}, tolerance(kit), name)


def test_a_far_token_decides_through_the_whole_model(kit):
    """One layer whose queries all look for the key of one token: the token at position 1, then 200 others.  With
    weights made so, the logits late in the sequence change by much when that token changes, in a prompt and in
    tokens decoded alone; the engine must follow the plain implementation in both."""
    cfg = {"architecture": "Zuzunex", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
           "layers": [_layer("attention", _plain(2, 1, 8, 8, 6.0, 40.0, (0.2, 50)), None)]}
    weights = pz.random_weights(cfg, 9)
    g = torch.Generator().manual_seed(3)

    def unit(n):
        v = torch.randn(n, generator=g)
        return v / v.norm()

    # Every embedding shares one direction, which the query projection picks up: all queries are large along the
    # first dimension of every head.  Tokens 7 and 8 are large, with opposite signs, along a second direction, which the
    # key projection puts on that same dimension: 7 draws every later query, 8 none.
    common, direction = unit(32), unit(32)
    direction = direction - (direction @ common) * common
    direction = direction / direction.norm()
    embed = 0.5 * torch.randn(50, 32, generator=g) + 2.0 * common
    embed[7], embed[8] = embed[7] + 6.0 * direction, embed[8] - 6.0 * direction
    weights["embed"] = embed
    weights["l0.norm1"], weights["l0.norm1.b"] = torch.ones(32), torch.zeros(32)
    weights["l0.mix.q"] = 0.05 * weights["l0.mix.q"]
    for head in range(2):
        weights["l0.mix.q"][head * 8] = 3.0 * common
    weights["l0.mix.k"][0] = direction  # the other rows of the key projection keep their size: the norm divides by all of them
    weights["l0.mix.sink"] = torch.tensor([0.5, -1.0])
    weights["l0.mix.g"] = 0.1 * weights["l0.mix.g"]
    weights["l0.mix.o"] = 3.0 * weights["l0.mix.o"]
    weights = {k: v.to(torch.bfloat16).float() for k, v in weights.items()}
    others = [t for t in helpers.random_ids(48, 230, 5) if t not in (7, 8)][:200]
    expected, got = {}, {}
    for far in (7, 8):
        ids = [others[0], far] + others[1:]
        expected[far] = plain_logits(cfg, weights, ids)
        steps = helpers.schedule_tail({"a": ids}, tail=40)
        engine = engine_of(cfg, weights, 8, kit, num_blocks=pages_needed(len(ids), 8), max_seqs=1)
        got[far] = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
        assert_close(got[far], {"a": expected[far]}, tolerance(kit), f"far token {far}")
    moved = row_errors(expected[7][-60:], expected[8][-60:])
    assert float(moved.min()) > 2 * tolerance(kit) and float(moved.median()) > 0.3, "the far token does not show in the late logits: the test's weights are too weak"


def test_long_decoding_beside_requests_that_come_and_go(kit):
    """Two tokens of prompt, then 150 tokens one by one beside another request that comes and goes twice over (its
    seat, pages and convolution state are used again)."""
    cfg, page, weights = model("small", kit)
    long_ids = helpers.random_ids(cfg["vocab"], 152, 5)
    other = helpers.random_ids(cfg["vocab"], 40, 6)
    steps = [{"step": 0, "entries": [{"id": "long", "tokens": long_ids[:2], "want": [0, 1]}], "end": []}]
    for at in range(2, len(long_ids)):
        entries = [{"id": "long", "tokens": [long_ids[at]], "want": [0]}]
        end = ["long"] if at == len(long_ids) - 1 else []
        if 40 <= at < 60:
            part = (at - 40) % 10
            entries.append({"id": f"o{(at - 40) // 10}", "tokens": other[4 * part : 4 * part + 4], "want": [3]})
            if part == 9:
                end.append(f"o{(at - 40) // 10}")
        steps.append({"step": at - 1, "entries": entries, "end": end})
    engine, _, _ = engine_for("small", kit, num_blocks=pages_needed(152, page) + pages_needed(40, page), max_seqs=2, max_model_len=160)
    got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
    want_other = plain_logits(cfg, weights, other)[3::4]
    assert_close(got, {"long": plain_logits(cfg, weights, long_ids), "o0": want_other, "o1": want_other}, tolerance(kit), "long")
    if kit.device.type == "cuda":  # steps of single tokens replayed the captured decode step
        assert engine.runner.use_graphs and engine.runner.graph_replays >= 100


@pytest.mark.parametrize("name", ["small", "awkward"])
def test_greedy_generation_through_the_scheduler(kit, name):
    """``Engine.run``: prompts cut into portions of five beside decoding requests, two seats for three requests, and
    one request sent back and recomputed; every token must be the plain implementation's arg-max (or a near tie)."""
    cfg, page, weights = model(name, kit)
    prompts = [helpers.random_ids(cfg["vocab"], n, 300 + n) for n in (17, 4, 26)]
    new_tokens = 12
    pool = pages_needed(max(len(p) for p in prompts) + new_tokens, page) * 2 + 1
    engine, _, _ = engine_for(name, kit, num_blocks=pool, max_seqs=2, prefill_chunk=5)
    sent_back, seen = [], []

    def on_token(request_id, token, finished):
        if request_id == "g0":
            seen.append(token)
            if len(seen) == 4:
                sent_back.append(engine.scheduler.force_preempt("g0"))

    results = engine.run([GenerateRequest(f"g{i}", p, new_tokens) for i, p in enumerate(prompts)], ignore_eos=True, on_token=on_token)
    assert sent_back == [True] and results[0].preemptions == 1
    for prompt, result in zip(prompts, results):
        assert len(result.token_ids) == new_tokens
        whole = prompt + result.token_ids[:-1]
        logits = plain_logits(cfg, weights, whole)[len(prompt) - 1 :]
        for index, token in enumerate(result.token_ids):
            slack = (2e-4 if kit.dtype == torch.float32 else 8e-2) * float(logits[index].std())
            assert float(logits[index, token]) >= float(logits[index].max()) - slack, f"{result.request_id}: output {index} is no arg-max"


# -- the command line and the trace runner, as a user runs them ---------------------------------------------
@pytest.mark.gpu
def test_command_line_and_trace_runner(tmp_path):
    """``init-random`` writes a Zuzunex folder from its configuration file, ``generate`` decodes greedily from it and
    ``bin/trace_run`` replays steps against it (a portion, then portions beside single tokens, then an ended request's
    seat used again): tokens and logits are the plain implementation's."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    from distie_b200.weights import ModelTensors

    ORACLE["stored"] = None  # both child processes run the float32 engine
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    config_file = tmp_path / "cfg.json"
    config_file.write_text(json.dumps(SMALL))
    folder = tmp_path / "model"
    subprocess.run([sys.executable, "-m", "distie_b200", "init-random", "--config", str(config_file), "--out", str(folder),
                    "--seed", "9", "--std", "0.3", "--dtype", "bfloat16"], check=True, env=env, cwd=root, timeout=600)
    stored = ModelTensors(str(folder))
    weights = {name: stored.tensor(name).float() for name in stored.keys()}
    prompt = helpers.random_ids(SMALL["vocab"], 9, 11)
    done = subprocess.run([sys.executable, "-m", "distie_b200", "generate", "--model", str(folder), "--dtype", "fp32",
                           "--prompt", " ".join(map(str, prompt)), "--max-new-tokens", "6", "--num-blocks", "8",
                           "--ignore-eos"], capture_output=True, text=True, env=env, cwd=root, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    tokens = json.loads(done.stdout)[0]["token_ids"]
    assert len(tokens) == 6
    logits = plain_logits(SMALL, weights, prompt + tokens[:-1])[len(prompt) - 1 :]
    for index, token in enumerate(tokens):
        assert float(logits[index, token]) >= float(logits[index].max()) - 2e-4 * float(logits[index].std())
    a, b, c = (helpers.random_ids(SMALL["vocab"], n, 50 + n) for n in (21, 13, 7))
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:17], "want": [0, 16]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[17:18], "want": [0]}, {"id": "b", "tokens": b[:6], "want": [5]}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[18:19], "want": [0]}, {"id": "b", "tokens": b[6:], "want": [6]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[19:20], "want": []}, {"id": "c", "tokens": c, "want": [6]}], "end": ["c"]},
        {"step": 4, "entries": [{"id": "a", "tokens": a[20:], "want": [0]}], "end": ["a"]},
    ]
    out_dir = tmp_path / "out"
    done = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out_dir),
                           "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps), env=env,
                          cwd=root, timeout=900, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done")] == [f"done {i}" for i in range(5)]
    la, lb, lc = (plain_logits(SMALL, weights, ids) for ids in (a, b, c))
    wanted = {0: torch.stack([la[0], la[16]]), 1: torch.stack([la[17], lb[5]]), 2: torch.stack([la[18], lb[12]]),
              3: lc[6:7], 4: la[20:21]}
    for step, want in wanted.items():
        have = torch.from_numpy(np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(want.shape[0], -1).copy())
        assert float(row_errors(have, want).max()) <= FP32_TOL, f"step {step}"
