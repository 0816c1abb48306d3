"""The Zururax decoder in the engine against the plain implementation (``plain_zururax``).

Every test that needs a kernel set takes the fixture ``kit``: the plain tensor-op set on the CPU
(``ref_kernels.RefKernels``, which checks the engine's bookkeeping: cache, batching, scheduling), and under
``-m gpu`` the CUDA sets in float32 and bfloat16.  Configurations are made here, with random weights; they
differ from one another in every size.  The plain implementation expands every head's keys and values from the
latent; the engine never does (it folds the queries into the latent's space), so the two share no formula.
"""

from __future__ import annotations

import copy

import pytest
import torch

import helpers
import plain_zururax as pz
from ref_kernels import RefKernels

from distie_b200.cache.manager import CacheManager, pages_needed
from distie_b200.config import ConfigError, EngineConfig, ZururaxConfig, get_architecture
from distie_b200.engine.batch import BatchEntry, lay_out, views
from distie_b200.engine.engine import Engine, GenerateRequest
from distie_b200.engine.trace_replay import TraceSession
from distie_b200.kernels.interface import KvSlot, RotaryTable
from distie_b200.models.decoder import model_tensor_specs
from distie_b200.parts import CacheNeed


def _mixer(heads, dim, rot, vdim, rank, q_rank, scale, base, kv_from=None):
    out = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "scale": scale,
           "rot": {"base": base, "dims": rot}}
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, scale, count, keep, ff, limit, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}},
            "expert": {"ff": ff, "limit": limit}, "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


# Small: every branch once.  Layer 0 owns a latent; layers 1 and 3 read it (two readers, one of them not the next
# layer, with head counts of their own); layer 2 owns another; a layer without a feed-forward; values of another size
# than keys; three groups of two experts of which two are kept.
SMALL = {
    "architecture": "Zururax", "vocab": 96, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "layers": [
        _layer(_mixer(3, 8, 4, 6, 20, 12, 0.3, 100.0), _dense(80)),
        _layer(_mixer(2, 12, 4, 10, 20, 16, 0.25, 100.0, kv_from=0), _moe(6, 2, 1.5, 3, 2, 24, 0.7, (40, 1.2))),
        _layer(_mixer(4, 8, 8, 8, 24, 12, 0.35, 5000.0), _moe(6, 2, 1.5, 3, 2, 24, 0.7, (40, 1.2))),
        _layer(_mixer(3, 8, 4, 6, 20, 12, 0.3, 100.0, kv_from=0), None),
    ],
}
# Awkward: a single head and five; sizes that are no powers of two and odd (a latent of 33, a rotated part of three
# pairs, a query latent of 7); no groups (one group, kept); groups of one expert; one chosen expert; as many chosen as
# eligible; no shared expert; a constant of 1 on the embedding and on the weights; pages of four tokens.
AWKWARD = {
    "architecture": "Zururax", "vocab": 101, "width": 72, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "layers": [
        _layer(_mixer(1, 24, 6, 10, 33, 7, 0.2, 1e6), _moe(5, 1, 1.0, 1, 1, 40, 2.5, None)),
        _layer(_mixer(5, 6, 2, 14, 9, 30, 0.4, 10.0), _moe(4, 2, 0.5, 4, 2, 16, 0.3, (8, 0.5))),
        _layer(_mixer(2, 16, 6, 3, 33, 11, 0.22, 1e6, kv_from=0), _dense(50)),
        _layer(_mixer(5, 10, 2, 4, 9, 5, 0.3, 10.0, kv_from=1), _moe(9, 3, 3.0, 3, 1, 8, 1.0, (24, 4.0))),
    ],
}
# Sizes of a real model's order: rows of 160 and 288 elements, steps of more than 128 tokens (in bfloat16 the
# tensor-core products run).
WIDE = {
    "architecture": "Zururax", "vocab": 500, "width": 256, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0},
    "layers": [
        _layer(_mixer(8, 64, 32, 64, 128, 96, 0.1, 10000.0), _moe(16, 4, 2.5, 4, 2, 64, 1.0, (128, 2.0))),
        _layer(_mixer(4, 32, 32, 48, 128, 64, 0.12, 10000.0, kv_from=0), _dense(384)),
        _layer(_mixer(2, 128, 32, 128, 256, 192, 0.08, 500000.0), _moe(8, 2, 1.0, 2, 1, 128, 1.5, (64, 1.0))),
    ],
}
CONFIGS = {"small": (SMALL, 8, 0), "awkward": (AWKWARD, 4, 1), "wide": (WIDE, 16, 2)}

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
    """``cfg`` with every router keeping all groups and choosing all experts: the weights still vary with the token,
    but no choice can be turned around by rounding."""
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            router = layer["mlp"]["router"]
            router["top"], router["groups"]["keep"] = router["experts"], router["groups"]["count"]
    return out


def model(name: str, kit=None):
    """The configuration, its page size and random weights.  For the bfloat16 engine the routers choose every expert
    (a choice that hangs on less than 16-bit activations can tell apart changes the token's row in the cache of every
    later layer); the float32 engines run the choices everywhere, and ``test_clear_choices_in_sixteen_bits`` runs
    them in bfloat16 where they are clear."""
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
    cfg = ZururaxConfig.from_dict(AWKWARD)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.embedding_scale, len(cfg.layers)) == (101, 72, 1e-6, 1.0, 4)
    first = cfg.layers[0].mixer
    assert (first.heads, first.dim, first.rot_dim, first.vdim, first.kv_rank, first.q_rank, first.kv_from) == (1, 24, 6, 10, 33, 7, None)
    assert (first.rot_base, first.rot_dims, first.scale) == (1e6, 6, 0.2)
    assert cfg.layers[2].mixer.kv_from == 0 and cfg.layers[3].mixer.kv_from == 1 and cfg.layers[2].mlp.ff == 50
    routed = cfg.layers[3].mlp
    assert (routed.experts, routed.top, routed.weight_scale, routed.group_count, routed.group_keep) == (9, 3, 3.0, 3, 1)
    assert (routed.ff, routed.limit, routed.shared_ff, routed.shared_limit) == (8, 1.0, 24, 4.0)
    assert cfg.layers[0].mlp.shared_ff is None and ZururaxConfig.from_dict(SMALL).layers[3].mlp is None
    for path, match in (
        (("layers", 1, "mixer", "kv_rank"), r"layers\[1\]\.mixer\.kv_rank"),
        (("layers", 0, "mixer", "rot", "base"), r"layers\[0\]\.mixer\.rot\.base"),
        (("layers", 1, "mlp", "router", "groups"), r"layers\[1\]\.mlp\.router\.groups"),
        (("layers", 2, "mlp", "expert", "limit"), r"layers\[2\]\.mlp\.expert\.limit"),
        (("embedding",), "embedding"),
        (("norm",), "norm"),
    ):
        broken = copy.deepcopy(SMALL)
        at = broken
        for key in path[:-1]:
            at = at[key]
        del at[path[-1]]
        with pytest.raises(ConfigError, match=match):
            ZururaxConfig.from_dict(broken)
    for change, match in (
        (lambda c: c["layers"][0].update(type="attention"), "attention"),
        (lambda c: c["layers"][0]["mlp"].update(kind="swiglu"), "swiglu"),
        (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "earlier"),
        (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "no latent of its own"),
        (lambda c: c["layers"][1]["mixer"].update(kv_rank=24), "kv_rank"),
        (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
        (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
        (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=4), "keep"),
    ):
        broken = copy.deepcopy(SMALL)
        change(broken)
        with pytest.raises(ConfigError, match=match):
            ZururaxConfig.from_dict(broken)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    cfg = CONFIGS[name][0]
    arch = get_architecture("Zururax")
    spec = arch.recipe(arch.config_cls.from_dict(cfg))
    specs = model_tensor_specs(spec)
    assert {s.name: tuple(s.shape) for s in specs} == {k: tuple(v) for k, v in pz.tensor_shapes(cfg).items()}
    # a layer that reads another's latent is a call that writes no cache and names the owner's slot
    owners = [i for i, layer in enumerate(cfg["layers"]) if layer["mixer"].get("kv_from") is None]
    for call, layer in zip(spec.order, cfg["layers"]):
        source = layer["mixer"].get("kv_from")
        assert call.writes_cache == (source is None) and call.cache_slot == owners.index(call.layer if source is None else source)


def test_random_model_folder_loads_by_its_config(tmp_path):
    from distie_b200.config import read_config
    from distie_b200.weights import write_random_model

    folder = write_random_model(str(tmp_path / "m"), SMALL, seed=3, std=0.1, norm_noise=0.05)
    arch, cfg = read_config(folder)
    assert arch.name == "Zururax" and cfg.width == 64
    engine = Engine.assemble(arch, cfg, folder, RefKernels(torch.float32),
                             EngineConfig(num_blocks=8, page_size=16, max_seqs=2, dtype="float32", device="cpu", decode_graphs=False))
    out = engine.generate([[1, 2, 3]], max_new_tokens=3, ignore_eos=True)
    assert len(out[0].token_ids) == 3


def test_a_latent_group_stores_one_row_per_token():
    need = CacheNeed(1, 24, value_dim=20, values_in_keys=True)
    assert need.row_elements == 24 and CacheNeed(2, 16).row_elements == 32
    cache = CacheManager({0: need, 1: need}, num_pages=6, page_size=4, max_seats=2, max_tokens_per_request=24,
                         device=torch.device("cpu"), dtype=torch.float32)
    group = cache.groups[0]
    slot = cache.kv_slot(0)
    assert slot.k.shape == (7, 1, 4, 24) and slot.v.shape == (7, 1, 4, 20)
    slot.k[2, 0, 1] = torch.arange(24.0)
    assert torch.equal(slot.v[2, 0, 1], torch.arange(20.0))  # a value is the head of its key's row: one store
    assert group.bytes_per_token(4) == 2 * 24 * 4



# -- each mechanism alone: ops of the kernel set against the plain functions ------------------------------------
def _latent_slot(kit, rank, rot, pages, page_size, table):
    """A cache slot of latent rows: one kv head, values the first ``rank`` columns of the keys."""
    dev = kit.device
    k = torch.zeros(pages, 1, page_size, rank + rot, dtype=kit.dtype, device=dev)
    return KvSlot(k, k[..., :rank], torch.tensor(table, dtype=torch.int32, device=dev), page_size, pages)


def _rows_of(kv, seat, positions):
    dev = kv.k.device
    pages = kv.block_table[seat, (positions // kv.page_size).to(dev)].long()
    return kv.k[pages, 0, (positions % kv.page_size).to(dev)]


@pytest.mark.parametrize("q_rank,rank,rot,heads,page,base", [(12, 20, 4, 3, 8, 100.0), (7, 33, 6, 1, 4, 1e6), (96, 128, 32, 8, 16, 1e4),
                                                             (5, 9, 2, 5, 4, 10.0), (192, 512, 64, 0, 16, 5e5)])
def test_latent_row_normed_rotated_and_stored(kit, q_rank, rank, rot, heads, page, base):
    """The stacked projection's accumulators (in slices) -> the normed query latent, and the token's one cache row:
    the normed latent beside the rotated key part; the gates' columns that follow are left alone."""
    g = torch.Generator().manual_seed(q_rank + rank)
    n, past, eps = 13, 2 * page + 3, 1e-5
    proj = torch.randn(n, q_rank + rank + rot + heads, generator=g) * 3
    q_w, kv_w = 1 + 0.2 * torch.randn(q_rank, generator=g), 1 + 0.2 * torch.randn(rank, generator=g)
    positions = torch.arange(past, past + n)
    p = proj.double()
    want_q = pz.rms_norm(p[:, :q_rank], q_w.double(), eps)
    want_c = pz.rms_norm(p[:, q_rank : q_rank + rank], kv_w.double(), eps)
    want_r = pz.rotate_pairs(p[:, q_rank + rank : q_rank + rank + rot], positions, base, rot)
    dev = kit.device
    width = pages_needed(past + n, page)
    kv = _latent_slot(kit, rank, rot, width + 1, page, [[-1] * width, list(range(width - 1, -1, -1))])
    step, _ = step_for(kit, [(1, [0] * n, past, ())])
    freqs = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float()
    table = RotaryTable(freqs.to(dev), rot, True)
    q_out = torch.empty(n, q_rank, dtype=kit.dtype, device=dev)
    kit.latent_kv_write(in_slices(proj.to(dev)), step, kv, table, q_rank, q_w.to(dev), rank, kv_w.to(dev), rot, eps, q_out)
    if hasattr(kit, "check_errors"):
        kit.check_errors()
    tol = 2e-5 if kit.dtype == torch.float32 else 1e-2
    _close(q_out, want_q, tol, "query latent")
    rows = _rows_of(kv, 1, positions)
    _close(rows[:, :rank], want_c, tol, "latent")
    _close(rows[:, rank:], want_r, tol, "rotated key part")
    assert kv.v.data_ptr() == kv.k.data_ptr()
    # a layer that reads another's rows: query columns only, and nothing is stored
    before = kv.k.clone()
    kit.latent_kv_write(proj[:, :q_rank].contiguous().to(dev), step, None, table, q_rank, q_w.to(dev), rank, None, rot, eps, q_out)
    _close(q_out, want_q, tol, "query latent alone")
    assert torch.equal(kv.k, before)


@pytest.mark.parametrize("heads,dim,rot,rank,base", [(3, 8, 4, 20, 100.0), (1, 24, 6, 33, 1e6), (8, 64, 32, 128, 1e4), (5, 6, 2, 9, 10.0),
                                                     (2, 128, 64, 512, 5e5)])
def test_queries_folded_into_the_latents_space(kit, heads, dim, rot, rank, base):
    g = torch.Generator().manual_seed(heads * dim)
    n, past = 9, 41
    q = torch.randn(n, heads * (dim + rot), generator=g)
    up_keys = torch.randn(heads, dim, rank, generator=g) / dim ** 0.5
    if kit.dtype != torch.float32:
        up_keys = up_keys.to(torch.bfloat16).float()
    positions = torch.arange(past, past + n)
    per_head = q.double().reshape(n, heads, dim + rot)
    plain = per_head[..., :dim]
    if kit.dtype != torch.float32:
        plain = plain.to(torch.bfloat16).double()
    want_folded = torch.einsum("thd,hdr->htr", plain, up_keys.double())
    want_rot = pz.rotate_pairs(per_head[..., dim:], positions, base, rot)
    dev = kit.device
    step, _ = step_for(kit, [(0, [0] * n, past, ())])
    freqs = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float()
    folded, rotated = kit.latent_queries(in_slices(q.to(dev)), up_keys.to(dev, kit.dtype), step, RotaryTable(freqs.to(dev), rot, True),
                                         heads, dim, rot)
    assert folded.shape == (heads, n, rank) and rotated.shape == (n, heads, rot)
    tol = 2e-5 if kit.dtype == torch.float32 else 1e-2
    _close(folded, want_folded, tol, "folded queries")
    _close(rotated, want_rot, tol, "rotated query part")
    # the fold keeps the score: folded . latent == q_plain . (W_uk latent)
    latent = torch.randn(rank, generator=g).double()
    keys = torch.einsum("hdr,r->hd", up_keys.double(), latent)
    _close(torch.einsum("htr,r->th", folded.double().cpu(), latent), torch.einsum("thd,hd->th", plain, keys),
           5e-5 if kit.dtype == torch.float32 else 3e-2, "score through the fold")


def _plain_latent_attention(folded, rotated, rows, rank, scale, sink):
    """``folded [h, n, rank]``, ``rotated [n, h, rot]``, ``rows [n, rank + rot]`` from position 0 -> ``[h, n, rank]``."""
    q = torch.cat([folded.transpose(0, 1), rotated], dim=-1)               # [n, h, rank + rot]
    heads = q.shape[1]
    k = rows[:, None, :].expand(-1, heads, -1)
    v = rows[:, None, :rank].expand(-1, heads, -1)
    return pz.sink_softmax_attention(q, k, v, scale, sink).transpose(0, 1)


@pytest.mark.parametrize("heads,rank,rot,page,n", [(3, 20, 4, 8, 90), (1, 33, 6, 4, 61), (8, 128, 32, 16, 300), (5, 9, 2, 4, 50),
                                                   (2, 512, 64, 16, 140), (16, 128, 0, 16, 70), (4, 48, 8, 8, 200), (3, 256, 64, 32, 330),
                                                   (2, 200, 24, 64, 270)])
def test_sink_softmax_over_latent_rows_with_keys_that_stand_out(kit, heads, rank, rot, page, n):
    """Rows go through pages handed out in reverse; attention runs in portions and token by token.  Every query looks
    for one direction of the latent and one of the rotated part.  The very first row, the rows on either side of every
    fourth page border and every seventh row carry one of them with a strength of their own, so one far row among
    hundreds decides most of an output.  Head 0's sink is far above every score (its output all but vanishes), the
    last head's far below (a plain softmax), the others' lie among the scores."""
    g = torch.Generator().manual_seed(rank + rot + n)
    rows = torch.randn(n, rank + rot, generator=g) * 0.5
    folded = torch.randn(heads, n, rank, generator=g) * 0.3
    rotated = torch.randn(n, heads, rot, generator=g) * 0.3
    a = torch.randn(rank, generator=g)
    a = a / a.norm()
    folded = folded + 3.0 * a
    marked = {0: 6.0}
    for border in range(4 * page, n, 4 * page):
        marked[border - 1], marked[border] = 4.0 + (border % 3), 5.5 - (border % 2)
    for j in range(3, n, 7):
        marked.setdefault(j, 2.0 + (j * 5 % 9) * 0.4)
    for j, strength in marked.items():
        rows[j, :rank] = strength * a + 0.1 * torch.randn(rank, generator=g)
    if rot:
        b = torch.randn(rot, generator=g)
        b = b / b.norm()
        rotated = rotated + 2.0 * b
        for j in range(5, n, 11):
            rows[j, rank:] = (3.0 + (j % 4)) * b
    sink = torch.randn(heads, generator=g) * 3 + 6
    sink[0] = 60.0
    sink[-1] = -60.0
    if kit.dtype != torch.float32:
        rows, folded, rotated = (t.to(torch.bfloat16).float() for t in (rows, folded, rotated))
    scale = 0.8
    want = _plain_latent_attention(folded.double(), rotated.double(), rows.double(), rank, scale, sink.double())
    dev = kit.device
    width = pages_needed(n, page)
    table = [[-1] * width, list(range(width - 1, -1, -1))]
    for cuts in ([1, 1, 2, page - 1, 1, 1, 2, 3 * page, 1, 1, 1, 4 * page + 1, 2], [n]):
        kv = _latent_slot(kit, rank, rot, width + 1, page, table)
        got, at = [], 0
        cuts = list(cuts)
        while at < n:
            count = min(cuts.pop(0) if cuts else 1, n - at)
            step, _ = step_for(kit, [(1, [0] * count, at, ())])
            at_rows = torch.arange(at, at + count)
            pages = kv.block_table[1, (at_rows // page).to(dev)].long()
            kv.k[pages, 0, (at_rows % page).to(dev)] = rows[at : at + count].to(dev, kit.dtype)
            out = torch.empty(heads, count, rank, dtype=kit.dtype, device=dev)
            kit.latent_attention(folded[:, at : at + count].contiguous().to(dev, kit.dtype),
                                 rotated[at : at + count].contiguous().to(dev, kit.dtype), step, kv, heads, rank, rot, scale,
                                 sink.to(dev), out)
            got.append(out.float().cpu())
            at += count
        if hasattr(kit, "check_errors"):
            kit.check_errors()
        have = torch.cat(got, dim=1)
        _close(have, want, 2e-5 if kit.dtype == torch.float32 else 3e-2, "attention over latent rows")
        if heads > 1:  # the sink took all of head 0's weight
            assert float(have[0].abs().max()) < 1e-6 * float(want.abs().max()) + 1e-12
    # without a sink: the plain softmax (the denominator holds the keys only)
    kit.latent_attention(folded[:, at - count : at].contiguous().to(dev, kit.dtype), rotated[at - count : at].contiguous().to(dev, kit.dtype),
                         step, kv, heads, rank, rot, scale, None, out)
    no_sink = _plain_latent_attention(folded.double(), rotated.double(), rows.double(), rank, scale, torch.full((heads,), -1e30, dtype=torch.float64))
    _close(out, no_sink[:, at - count : at], 2e-5 if kit.dtype == torch.float32 else 3e-2, "no sink")


@pytest.mark.parametrize("heads,rank,vdim", [(3, 20, 6), (1, 33, 10), (8, 128, 64), (5, 9, 14), (2, 256, 128)])
def test_values_from_the_mixed_latents_and_gated_heads(kit, heads, rank, vdim):
    g = torch.Generator().manual_seed(heads + rank + vdim)
    n = 11
    mixed = torch.randn(heads, n, rank, generator=g)
    up_values = torch.randn(heads, rank, vdim, generator=g) / rank ** 0.5
    gate = torch.randn(n, heads + 3, generator=g) * 2
    if kit.dtype != torch.float32:
        mixed, up_values = mixed.to(torch.bfloat16).float(), up_values.to(torch.bfloat16).float()
    plain = torch.einsum("htr,hrv->thv", mixed.double(), up_values.double())
    want = plain * torch.sigmoid(gate.double()[:, 3:, None])
    dev = kit.device
    tol = 2e-5 if kit.dtype == torch.float32 else 2e-2
    gates = in_slices(gate.to(dev))[..., 3:]  # the last columns of a wider split product, as the mixer passes them
    out = kit.latent_values(mixed.to(dev, kit.dtype), up_values.to(dev, kit.dtype), gates, heads, vdim)
    assert out.shape == (n, heads * vdim) and out.dtype == kit.dtype
    _close(out, want.reshape(n, -1), tol, "gated heads")
    out = kit.latent_values(mixed.to(dev, kit.dtype), up_values.to(dev, kit.dtype), None, heads, vdim)
    _close(out, plain.reshape(n, -1), tol, "no gate")


def _plain_choice(scores, top, count, keep):
    return [pz.choose_experts(scores[t], top, count, keep) for t in range(scores.shape[0])]


@pytest.mark.parametrize("experts,top,count,keep,width", [(6, 2, 3, 2, 64), (9, 3, 3, 1, 72), (4, 2, 4, 2, 40), (5, 1, 1, 1, 48),
                                                          (16, 4, 4, 2, 256), (64, 8, 8, 3, 128), (12, 6, 2, 1, 56), (8, 8, 4, 4, 32)])
def test_experts_chosen_among_the_best_groups(kit, experts, top, count, keep, width):
    """Scores on a grid of distinct values (no choice hangs on rounding).  Some tokens are made so that the group
    rule shows: the expert with the largest score of all sits in a group whose second score is small, beside groups
    of two middling scores, and must not be chosen when its group falls out."""
    g = torch.Generator().manual_seed(experts * 7 + top)
    tokens = min(60, width)
    size = experts // count
    levels = torch.linspace(-2.5, 2.5, experts * 2)
    table = torch.stack([levels[torch.randperm(experts * 2, generator=g)[:experts]] for _ in range(tokens)])
    if count > keep and size >= 2:
        for t in range(0, tokens, 3):
            order = torch.argsort(table[t], descending=True)
            lone = int(torch.randint(0, count, (1,), generator=g))
            row = torch.empty(experts)
            mids = iter(order[1 : 1 + 2 * (count - 1)].tolist())
            rest = iter(order[1 + 2 * (count - 1) :].tolist())
            for group in range(count):
                members = list(range(group * size, (group + 1) * size))
                if group == lone:
                    row[members[0]] = table[t, order[0]]
                    for e in members[1:]:
                        row[e] = table[t, order[-1 - (e - members[0])]] - 3.0
                else:
                    row[members[0]], row[members[1]] = table[t, next(mids)], table[t, next(mids)]
                    for e in members[2:]:
                        row[e] = table[t, next(rest)] - 6.0
            table[t] = row
    # every token is a unit vector of its own, so that the router's logits are the rows of the table made here
    x = torch.eye(tokens, width)
    router = torch.zeros(experts + 2, width)
    router[:, :tokens] = torch.cat([table, torch.randn(tokens, 2, generator=g)], 1).T
    x, router = x.to(torch.bfloat16).float(), router.to(torch.bfloat16).float()
    logits = x.double() @ router.double().T
    scores = torch.sigmoid(logits[:, :experts])
    margins = torch.tensor([pz.choice_margin(scores[t], top, count, keep) for t in range(tokens)])
    clear = margins > 1e-3
    assert int(clear.sum()) >= tokens // 2
    want = _plain_choice(scores, top, count, keep)
    dev = kit.device
    scale = 1.5
    ids, weights, extra = kit.route_top(x.to(dev, kit.dtype), router.to(dev, kit.dtype), top, "sigmoid", (count, keep), scale, 2)
    assert ids.dtype == torch.int32 and ids.shape == (tokens, top) and extra.shape == (tokens, 2) and extra.dtype == torch.float32
    for t in range(tokens):
        if clear[t]:
            assert ids[t].cpu().tolist() == want[t], f"token {t}"
            _close(weights[t], scale * scores[t, want[t]], 1e-5, "weights: the chosen scores times the constant")
    _close(extra, logits[:, experts:], 1e-5, "the rows below the experts' are logits of their own")
    if count > keep and size >= 2:  # the rule bit: somewhere the best expert of all was left out
        assert any(clear[t] and int(scores[t].argmax()) not in want[t] for t in range(0, tokens, 3))
    # without groups and rows to spare: the plain choice of the largest scores
    ids, weights = kit.route_top(x.to(dev, kit.dtype), router[:experts].contiguous().to(dev, kit.dtype), top, "sigmoid", None, 1.0)[:2]
    for t in range(tokens):
        if pz.choice_margin(scores[t], top, 1, 1) > 1e-3:
            assert ids[t].cpu().tolist() == pz.choose_experts(scores[t], top, 1, 1)


@pytest.mark.parametrize("width,ff,limit,tokens", [(64, 24, 0.7, 9), (72, 40, 2.5, 70), (256, 128, 1.0, 150), (40, 8, 0.3, 3)])
def test_capped_gated_layer_and_the_row_gate(kit, width, ff, limit, tokens):
    """Inputs large enough that the cap bites on both sides of the up projection and above on the gate."""
    g = torch.Generator().manual_seed(width + ff)
    x = torch.randn(tokens, width, generator=g) * 1.5
    w = {"gate": torch.randn(ff, width, generator=g) / width ** 0.5, "up": torch.randn(ff, width, generator=g) / width ** 0.5,
         "down": torch.eye(ff)}
    row_gate = torch.randn(tokens, 5, generator=g) * 2
    x, w = x.to(torch.bfloat16).float(), {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    wd = {k: v.double() for k, v in w.items()}
    hidden = pz.capped_expert(x.double(), wd, "", limit)  # the down map is the identity: the hidden layer itself
    both = x.double() @ torch.cat([wd["gate"], wd["up"]]).T
    assert bool((both[:, :ff] > limit).any()) and bool((both[:, ff:] > limit).any()) and bool((both[:, ff:] < -limit).any())
    dev = kit.device
    tol = 2e-5 if kit.dtype == torch.float32 else 2e-2
    stacked = torch.cat([w["gate"], w["up"]]).to(dev, kit.dtype)
    out = kit.linear_glu(x.to(dev, kit.dtype), stacked, limit, None)
    assert out.shape == (tokens, ff) and out.dtype == kit.dtype
    _close(out, hidden, tol, "capped hidden layer")
    gated = kit.linear_glu(x.to(dev, kit.dtype), stacked, limit, in_slices(row_gate.to(dev))[..., 4:5])
    _close(gated, hidden * torch.sigmoid(row_gate.double()[:, 4:5]), tol, "times the sigmoid of the row's logit")
    silu = kit.linear_glu(x.to(dev, kit.dtype), stacked, None, None)
    _close(silu, torch.nn.functional.silu(both[:, :ff]) * both[:, ff:], tol, "no limit: SwiGLU")
    # the squared ReLU of a plain hidden layer
    act = kit.linear_act(x.to(dev, kit.dtype), w["up"].to(dev, kit.dtype), "relu2")
    _close(act, torch.relu(both[:, ff:]) ** 2, tol, "squared ReLU")
    assert bool((act == 0).any()) and bool((act > 0).any())


@pytest.mark.parametrize("experts,top,width,ff,limit", [(6, 2, 64, 24, 0.7), (5, 1, 72, 40, 2.5), (16, 4, 256, 64, 1.0), (9, 3, 40, 8, 0.4),
                                                        (4, 3, 320, 136, 5.0)])
def test_capped_experts_weighted_on_their_output(kit, experts, top, width, ff, limit):
    g = torch.Generator().manual_seed(experts + width)
    tokens = 70 if width < 256 else 150 if width < 320 else 400  # (from 512 pairs on, bfloat16 takes the tile kernel)
    x = torch.randn(tokens, width, generator=g) * 1.5
    w = {}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"] = (torch.randn(ff, width, generator=g) / width ** 0.5 for _ in range(2))
        w[f"e{e}.down"] = torch.randn(width, ff, generator=g) / ff ** 0.5
    x, w = x.to(torch.bfloat16).float(), {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    x[5] = x[4]
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(tokens)]).to(torch.int32)
    ids[5] = ids[4]
    weights = torch.rand(tokens, top, generator=g) * 2
    weights[5] = weights[4]
    wd = {k: v.double() for k, v in w.items()}
    want = torch.zeros(tokens, width, dtype=torch.float64)
    for t in range(tokens):
        for e, s in zip(ids[t].tolist(), weights[t].double()):
            want[t] += s * pz.capped_expert(x[t : t + 1].double(), wd, f"e{e}.", limit)[0]
    dev = kit.device
    gate_up = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(experts)]).to(dev, kit.dtype)
    down = torch.stack([w[f"e{e}.down"] for e in range(experts)]).to(dev, kit.dtype)
    out = kit.routed_swiglu(x.to(dev, kit.dtype), ids.to(dev), weights.to(dev), gate_up, down, False, limit)
    assert out.shape == (top, tokens, width) and out.dtype == torch.float32
    total = out.sum(0)
    _close(total, want, 2e-5 if kit.dtype == torch.float32 else 2e-2, "capped experts")
    assert torch.equal(total[5], total[4])
    few = kit.routed_swiglu(x[:3].to(dev, kit.dtype), ids[:3].contiguous().to(dev), weights[:3].contiguous().to(dev), gate_up, down, False, limit)
    _close(few.sum(0), total[:3].double().cpu(), 1e-5 if kit.dtype == torch.float32 else 1e-2, "few rows against many")


# -- each kind of layer alone in a model, then all of them ---------------------------------------------------
ALONE = {
    "latent": [_layer(_mixer(3, 8, 6, 10, 14, 9, 0.4, 300.0), None)],
    "reader": [_layer(_mixer(2, 8, 4, 8, 12, 6, 0.3, 50.0), None), _layer(_mixer(4, 6, 4, 5, 12, 10, 0.5, 50.0, kv_from=0), None)],
    "dense": [_layer(_mixer(1, 8, 2, 8, 8, 8, 0.3, 50.0), _dense(44))],
    "routed": [_layer(_mixer(1, 8, 2, 8, 8, 8, 0.3, 50.0), _moe(8, 3, 2.0, 4, 2, 20, 0.6, (28, 0.9)))],
}


@pytest.mark.parametrize("kind", list(ALONE))
def test_one_layer_of_a_kind_prefill_against_single_tokens(kit, kind):
    cfg = {"architecture": "Zururax", "vocab": 60, "width": 56, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "layers": copy.deepcopy(ALONE[kind])}
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
    """The bfloat16 engine with routers that choose a few experts of a few groups, on prompts whose every choice is
    clear (found by trying seeds against the plain implementation): whole prompts, prefill against single tokens,
    portions."""
    from distie_b200.kernels import make_kernels

    kit = make_kernels(torch.bfloat16, "cuda:0")
    ORACLE["stored"] = torch.bfloat16
    cfg, page, weights = copy.deepcopy(SMALL), 8, pz.random_weights(SMALL, 0)
    requests = {}
    for seed in range(400, 2400):
        ids = helpers.random_ids(cfg["vocab"], 12, seed)
        margins = []
        plain_logits(cfg, weights, ids, margins)
        if float(torch.stack(margins).min()) >= 0.03:
            requests[f"c{len(requests)}"] = ids
            if len(requests) == 3:
                break
    assert len(requests) == 3, "no prompts with clear choices among the seeds tried"
    expected = {rid: plain_logits(cfg, weights, ids) for rid, ids in requests.items()}
    for schedule in (helpers.schedule_whole, lambda r: helpers.schedule_tail(r, tail=9), helpers.schedule_portions):
        steps = schedule(requests)
        engine = engine_of(cfg, weights, page, kit, num_blocks=8, max_seqs=2)
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
    peak and three seats, so that pages and seats are used again."""
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
    # one cache group per latent of its own, one row per token; layers that read another's add none
    owners = [layer for layer in cfg["layers"] if layer["mixer"].get("kv_from") is None]
    assert sorted(g.need.head_dim for g in engine.cache.groups) == sorted(l["mixer"]["kv_rank"] + l["mixer"]["rot_dim"] for l in owners)
    if kit.device.type == "cuda":
        ran = kit.kernel_counts
        assert (ran.get("latent_attention") or ran.get("latent_attention_mma")) and ran.get("latent_kv_write") and ran.get("routed_swiglu") and ran.get("glu_act")


@pytest.mark.parametrize("name", ["small", "awkward"])
def test_cuts_at_around_and_across_page_borders(kit, name):
    """The first tokens one by one; portions that end just before, at and just after page borders; two tokens at a
    time across one; then single tokens across the next ones."""
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
    """One layer whose queries all look for the latent of one token: the token at position 1, then 200 others.  With
    weights made so, the logits late in the sequence change by much when that token changes, in a prompt and in
    tokens decoded alone; the engine must follow the plain implementation in both."""
    cfg = {"architecture": "Zururax", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
           "layers": [_layer(_mixer(2, 8, 4, 8, 16, 8, 1.0, 10000.0), None)]}
    weights = pz.random_weights(cfg, 9)
    g = torch.Generator().manual_seed(3)

    def unit(n):
        v = torch.randn(n, generator=g)
        return v / v.norm()

    # Every embedding shares one direction, which the query latent picks up: all queries are large along the first
    # plain dimension of every head.  Tokens 7 and 8 are large, with opposite signs, along a second direction, which
    # the key/value latent picks up and the keys' map puts on that same dimension: 7 draws every later query, 8 none.
    common, direction = unit(32), unit(32)
    direction = direction - (direction @ common) * common
    direction = direction / direction.norm()
    embed = 0.5 * torch.randn(50, 32, generator=g) + 2.0 * common
    embed[7], embed[8] = embed[7] + 6.0 * direction, embed[8] - 6.0 * direction
    weights["embed"] = embed
    weights["l0.norm1"] = torch.ones(32)
    weights["l0.mix.dq"][0] = 3.0 * common
    weights["l0.mix.dq.norm"] = torch.ones(8)
    weights["l0.mix.dkv"][0] = 3.0 * direction
    weights["l0.mix.dkv.norm"] = torch.ones(16)
    weights["l0.mix.uq"], weights["l0.mix.uk"] = 0.1 * weights["l0.mix.uq"], 0.1 * weights["l0.mix.uk"]
    for head in range(2):
        weights["l0.mix.uq"][head * 12, 0] = 3.0
        weights["l0.mix.uk"][head * 8, 0] = 3.0
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
    assert float(moved.min()) > 2 * tolerance(kit) and float(moved.median()) > 0.5, "the far token does not show in the late logits: the test's weights are too weak"


def test_long_decoding_beside_requests_that_come_and_go(kit):
    """Two tokens of prompt, then 150 tokens one by one beside another request that comes and goes twice over (its
    seat and pages are used again)."""
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
    """``init-random`` writes a Zururax folder from its configuration file, ``generate`` decodes greedily from it and
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
    prompt = helpers.random_ids(SMALL["vocab"], 19, 41)
    proc = subprocess.run([sys.executable, "-m", "distie_b200", "generate", "--model", str(folder), "--dtype", "fp32",
                           "--prompt", " ".join(map(str, prompt)), "--max-new-tokens", "8", "--num-blocks", "8",
                           "--ignore-eos"], capture_output=True, text=True, env=env, cwd=root, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    tokens = json.loads(proc.stdout)[0]["token_ids"]
    logits = plain_logits(SMALL, weights, prompt + tokens[:-1])[len(prompt) - 1 :]
    for index, token in enumerate(tokens):
        assert float(logits[index, token]) >= float(logits[index].max()) - 2e-4 * float(logits[index].std())

    a, b = helpers.random_ids(SMALL["vocab"], 40, 42), helpers.random_ids(SMALL["vocab"], 30, 43)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:25], "want": [0, 24]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[25:26], "want": [0]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[7:], "want": [22]}, {"id": "a", "tokens": a[26:], "want": [13]}], "end": ["a", "b"]},
        {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [29]}], "end": ["c"]},
    ]
    for dtype, tol in (("float32", FP32_TOL), ("bfloat16", BF16_TOL)):
        out = tmp_path / f"out_{dtype}"
        proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                               "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                              text=True, env=env, cwd=root, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [line for line in proc.stdout.splitlines() if line.startswith("done")] == [f"done {i}" for i in range(4)]
        if dtype == "bfloat16":
            continue  # a router's close call may go either way in 16 bits; the runs above hold the bfloat16 engine to the oracle
        full_a, full_b = plain_logits(SMALL, weights, a), plain_logits(SMALL, weights, b)
        want = {0: full_a[[0, 24]], 1: torch.stack([full_a[25], full_b[6]]), 2: torch.stack([full_b[29], full_a[39]]), 3: full_b[[29]]}
        for step, rows in want.items():
            got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(rows.shape))
            assert float(row_errors(got, rows).max()) <= tol, f"step {step}"
