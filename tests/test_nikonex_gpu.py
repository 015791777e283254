"""The Nikonex decoder through the engine against its plain implementation (tests/plain/nikonex_plain.py):
every mechanism alone, whole prompts against token-by-token decoding, prompts in portions, unequal batches,
slots, pages and states that are used again, keys at the edges of windows and pages, the first tokens of a
sequence, long decoding, sizes that the fast kernels take and sizes that they do not, and greedy generation
through the engine's own entry point.  The tests write their own weights and inputs (matrices of unit gain, a
router whose scores spread, loud tokens whose rotated key part dwarfs every other score) so that a window that is
one token off, a lost state or a group that is scored wrongly leaves a mark far above rounding."""
import json
import math
import os

import numpy as np
import pytest
import torch

from tests import traces
from tests.plain import nikonex_plain as P
from tests.tiny import TOL, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, scale, base=1e4, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if rot_dim:
        m["rot"] = {"dims": rot_dim, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = scaling
    if window:
        m["mask"] = {"size": window}
    return m


def retention(heads, dim, vdim, decay, rot_dims=0, base=1e4):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return m


def moe(experts, top, ff, groups=None, scale=None, shared=0):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        router["scale"] = scale
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(kind, mx, mlp):
    return {"type": kind, "mixer": mx, "mlp": mlp}


RAMP = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
# MIXED: value heads smaller and larger than keys, cached rows of 48 and 72 elements, a retention layer whose rotation
# covers part of a head, a layer without a feed-forward, groups of which two of three stay, a shared expert of twice
# the experts' size (rides with them) and one of another size (runs beside them), a window of one key
MIXED = {"architecture": "Nikonex", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 0.4,
         "layers": [layer("latent_attention", latent(3, 24, 8, 20, 36, 40, 37, 0.21, 5000.0, RAMP), moe(6, 2, 40, (3, 2), 2.5, 56)),
                    layer("retention", retention(2, 24, 40, [0.9, 0.995], 16, 1000.0), None),
                    layer("retention", retention(3, 16, 16, [0.5, 0.97, 1.0], 16), moe(8, 3, 24, (4, 2), 0.7, 48)),
                    layer("latent_attention", latent(2, 16, 24, 40, 20, 48, 1, 0.3), moe(4, 1, 32, (2, 1), None, 0)),
                    layer("latent_attention", latent(4, 8, 16, 8, 64, 24, 64, 0.15, 1e6, dict(RAMP, factor=16.0, original=32)), None)]}
# ODD: a width that is no multiple of 8 (products on CUDA cores), one head, every expert chosen, no groups, no shared
# expert, no window, no frequency scaling, retention that does not rotate, no factor on the updates
ODD = {"architecture": "Nikonex", "vocab": 97, "width": 100, "norm": {"eps": 1e-6},
       "layers": [layer("retention", retention(1, 20, 12, [0.8]), moe(3, 3, 28)),
                  layer("latent_attention", latent(1, 20, 6, 12, 10, 30, 0, 0.2), moe(5, 2, 12, (5, 2), 3.0, 20)),
                  layer("retention", retention(5, 8, 12, [0.99, 0.9, 0.7, 0.3, 0.0], 4, 50.0), None)]}
# FAST: cached rows of 128 and 64 elements (the tensor-core attention kernels), windows across several pages, widths
# the tensor-core products take, retention heads of 64
FAST = {"architecture": "Nikonex", "vocab": 512, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.8,
        "layers": [layer("latent_attention", latent(8, 32, 64, 32, 64, 64, 300, 0.1, 25000.0, dict(RAMP, original=256)), moe(8, 3, 64, (2, 1), 1.5, 128)),
                   layer("retention", retention(2, 64, 64, [0.98, 0.999], 64, 1e5), moe(12, 2, 48, (3, 1), 2.0, 80)),
                   layer("latent_attention", latent(4, 64, 16, 48, 96, 48, 70, 0.09), moe(4, 2, 128)),
                   layer("retention", retention(4, 32, 32, [0.9, 0.95, 0.99, 0.995], 16), None)]}
CONFIGS = {"mixed": (MIXED, 3), "odd": (ODD, 5), "fast": (FAST, 7)}


def write_model(folder: str, raw: dict, seed: int) -> str:
    """A model folder with weights of the test's own making: matrices N(0, 1/in) so that activations keep their
    size from layer to layer, norm weights around one, a router of gain 3, a gate vector of gain 2."""
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.weights import model_param_specs
    from odin_infer_b200.weights.safetensors_io import write_safetensors
    cfg = config_from_dict(raw)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    gen = torch.Generator().manual_seed(seed)
    specs = model_param_specs(cfg)

    def make(name):
        shape = next(s.concrete_shape for s in specs if s.name == name)
        r = torch.randn(shape, generator=gen)
        if name.endswith(("norm1", "norm2", "final.norm")):
            t = 1.0 + 0.3 * r
        elif name.endswith(".norm"):
            t = 1.0 + 0.2 * r
        elif name == "embed":
            t = r
        elif name.endswith("router"):
            t = 3.0 * r / math.sqrt(shape[1])
        elif name.endswith(".sg"):
            t = 2.0 * r / math.sqrt(shape[1])
        elif name.endswith((".o", "down")):
            t = 0.5 * r / math.sqrt(shape[1])
        else:
            t = r / math.sqrt(shape[1])
        return t.to(torch.bfloat16)
    write_safetensors(os.path.join(folder, "model.safetensors"), [(s.name, torch.bfloat16, s.concrete_shape) for s in specs], make)
    return folder


_folders = {}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    if not _folders:
        base = tmp_path_factory.mktemp("nikonex")
        for name, (raw, seed) in CONFIGS.items():
            _folders[name] = write_model(os.path.join(str(base), name), raw, seed)
    return _folders


_plain = {}


def plain_logits(folder, tokens, rounded=False):
    key = (folder, tuple(tokens), rounded)
    if key not in _plain:
        cfg, w = P.read_model_folder(folder, F64)
        _plain[key] = P.forward(cfg, w, tokens, rnd=P.to_bfloat16_and_back if rounded else (lambda t: t)).numpy()
    return _plain[key]


def engine_for(folder, dtype, max_tokens=4096, max_ctx=1024, graphs=True):
    from odin_infer_b200 import Engine, Engine_Opts
    return Engine.load(folder, Engine_Opts(max_ctx=max_ctx, max_tokens=max_tokens, dtype=dtype, verbose=False,
                                           cuda_graphs=graphs))


def replay(engine, recs):
    from odin_infer_b200.engine.trace import replay as run
    return run(engine, recs)


def requests_for(raw, lengths, seed=0):
    return {f"r{i}": random_tokens(n, raw["vocab"], seed + i) for i, n in enumerate(lengths)}


# The 32-bit engine is held to the tolerance everywhere.  In bfloat16 the yardstick is what rounding alone does to
# this model and these tokens: the plain implementation run once more with everything that a 16-bit engine stores in
# 16 bits rounded to bfloat16.  A router's close call then falls the other way for some token, its update differs by
# an expert's share, and later tokens see that through the mixers: the error is no smooth function of the position,
# and the engine's close calls are not the plain implementation's.  So a position's limit is the tolerance or three
# times the rounding's own error there, one position in ten may be over it, the median stays within twice the
# rounding's median (or a quarter of the tolerance), and no position is wild.  Every kernel alone is held to its
# tolerance in bfloat16 further down, with choices that are no close calls.
def check_rows(got: dict, folder, requests, dtype):
    for rid, rows in got.items():
        n = rows.shape[0]
        ref = plain_logits(folder, requests[rid])[:n]
        top = max(np.abs(ref).max(), 1e-30)
        err = np.abs(rows.astype(np.float64) - ref).max(axis=1) / top
        if dtype == "float32":
            assert err.max() <= TOL[dtype], f"{rid}: relative error {err.max():.3e} > {TOL[dtype]:.1e} at {int(err.argmax())}"
            continue
        noise = np.abs(plain_logits(folder, requests[rid], rounded=True)[:n] - ref).max(axis=1) / top
        over = int((err > np.maximum(TOL[dtype], 3.0 * noise)).sum())
        mid = max(TOL[dtype] / 4, 2.0 * float(np.median(noise)))
        assert over <= max(2, n // 10) and err.max() <= max(2.0, 3.0 * noise.max()) and np.median(err) <= mid, \
            (f"{rid}: {over} of {n} positions over their limit, median {np.median(err):.3e} (rounding alone "
             f"{np.median(noise):.3e}), worst {err.max():.3e} at {int(err.argmax())} (rounding alone {noise.max():.3e})")


# --------------------------------------------------------------------------------------
# the whole model in every cut
# --------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_and_one_by_one(folders, name, dtype):
    """Whole prompts (across several windows and pages), then the same with the last tokens one by one, so that
    decoding walks over window and page borders and the recurrent state passes from the prompt's kernel to the
    single-token one; the first tokens of a sequence alone (prompts of 1 and 2)."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [1, 2, 131, 330])
    engine = engine_for(folders[name], dtype)
    check_rows(traces.collect(traces.whole(reqs), replay(engine, traces.whole(reqs))), folders[name], reqs, dtype)
    recs = traces.tail_one_by_one(reqs, tail=70)
    check_rows(traces.collect(recs, replay(engine, recs)), folders[name], reqs, dtype)
    engine.cache.check()
    assert all(g.pool.n_held == 0 for g in engine.cache.groups.values())
    engine.destroy()


def portions(requests, sizes):
    """Each request alone, fed in portions of the given sizes in turn (the last one takes what is left)."""
    recs, n = [], 0
    for rid, toks in requests.items():
        at, i = 0, 0
        while at < len(toks):
            k = min(sizes[i % len(sizes)], len(toks) - at)
            recs.append({"step": n, "entries": [{"id": rid, "tokens": toks[at:at + k], "want": list(range(k))}],
                         "end": [rid] if at + k == len(toks) else []})
            at, i, n = at + k, i + 1, n + 1
    return recs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,sizes", [("mixed", (2, 35, 3, 64)), ("odd", (17, 2, 2, 90)), ("fast", (130, 2, 70, 1, 129)),
                                        ("mixed", (2,))])
def test_prompts_in_portions(folders, name, sizes, dtype):
    """Portions of several sizes, down to two tokens: a portion's first tokens see the window's keys of the portions
    before it and start from the state that the portion before it left."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [150, 41] if sizes == (2,) else [333, 77], seed=10)
    engine = engine_for(folders[name], dtype)
    recs = portions(reqs, sizes)
    check_rows(traces.collect(recs, replay(engine, recs)), folders[name], reqs, dtype)
    engine.destroy()


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batches_and_reuse(folders, name, dtype, graphs):
    """Batches of unequal requests, batch after batch in a cache that holds one batch only, so that every slot, every
    page and every slot's recurrent state is used again (a state that is not cleared shows in the next request);
    shorter requests end earlier."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [5, 180, 66, 1, 129, 40, 97, 260, 3], seed=20)
    recs = traces.batches(reqs, 3, first_part=lambda n: max(1, n - 9))
    engine = engine_for(folders[name], dtype, max_tokens=traces.max_live_tokens(recs) + 64, graphs=graphs)
    check_rows(traces.collect(recs, replay(engine, recs)), folders[name], reqs, dtype)
    engine.cache.check()
    engine.destroy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_requests_join_a_running_batch(folders, dtype):
    raw = CONFIGS["mixed"][0]
    reqs = requests_for(raw, [60, 45, 90, 30, 75], seed=30)
    recs = traces.joining(reqs)
    engine = engine_for(folders["mixed"], dtype)
    check_rows(traces.collect(recs, replay(engine, recs)), folders["mixed"], reqs, dtype)
    engine.destroy()


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_cuts_agree_in_32_bit(folders, name):
    """In 32-bit a position's logits agree to rounding whole, in portions, one by one and in a batch: the attention
    layers and the experts give the same bits in every cut, the recurrent state is carried in another order of sums
    when a prompt is cut (blocks of tokens), which costs the last bits."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [140, 59], seed=40)
    engine = engine_for(folders[name], "float32")
    ref = traces.collect(traces.whole(reqs), replay(engine, traces.whole(reqs)))
    for recs in (portions(reqs, (3, 50, 2)), traces.tail_one_by_one(reqs, tail=25), traces.batches(reqs, 2)):
        got = traces.collect(recs, replay(engine, recs))
        for rid in reqs:
            top = np.abs(ref[rid]).max()
            assert np.abs(got[rid] - ref[rid]).max() <= 2e-6 * top, rid
    # a batch is the same bits as each request alone in the same cut
    alone = traces.collect(traces.batches(reqs, 1), replay(engine, traces.batches(reqs, 1)))
    both = traces.collect(traces.batches(reqs, 2), replay(engine, traces.batches(reqs, 2)))
    for rid in reqs:
        assert np.array_equal(alone[rid], both[rid]), rid
    engine.destroy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "fast"])
def test_long_decoding(folders, name, dtype):
    """Three hundred tokens decoded one by one after a short prompt: every window passes over decoded tokens many
    times, the pages that fall out of a window go back to the pool, and the state is carried three hundred times."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [330, 318], seed=50)
    recs = traces.batches(reqs, 2, first_part=lambda n: 12)
    engine = engine_for(folders[name], dtype)
    check_rows(traces.collect(recs, replay(engine, recs)), folders[name], reqs, dtype)
    assert all(g.pool.n_held == 0 for g in engine.cache.groups.values())
    engine.destroy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt(folders, dtype):
    """A prompt of 1,100 tokens whole, and with its last 40 tokens one by one: windows many pages back from the start,
    a recurrence over many blocks of tokens, experts with several tiles of rows each."""
    raw = CONFIGS["fast"][0]
    reqs = requests_for(raw, [1100], seed=70)
    engine = engine_for(folders["fast"], dtype, max_tokens=2048, max_ctx=1280)
    for recs in (traces.whole(reqs), traces.tail_one_by_one(reqs, tail=40)):
        check_rows(traces.collect(recs, replay(engine, recs)), folders["fast"], reqs, dtype)
    engine.cache.check()
    engine.destroy()


def test_latent_rows_share_storage_and_windows_give_pages_back(folders):
    """Latent layers with equal rows and windows share a group of the cache (a line each); a windowed group holds
    only the pages that its window still reaches; retention layers hold no pages at all."""
    from odin_infer_b200 import StepEntry
    engine = engine_for(folders["mixed"], "float32")
    shapes = sorted((g.request.head_dim, g.request.window, g.n_lines) for g in engine.cache.groups.values())
    assert shapes == [(40, 64, 1), (48, 37, 1), (72, 1, 1)], shapes
    assert all(g.request.shared_kv for g in engine.cache.groups.values())
    slot = engine.take_slot()
    engine.step([StepEntry(slot, random_tokens(200, 211, 1), [199])])
    held = {g.request.window: g.pool.n_held for g in engine.cache.groups.values()}
    # the next query sits at position 200: it sees from 200 - window + 1 on; pages are 64 tokens
    assert held == {37: 2, 64: 2, 1: 1}, held
    engine.give_back_slot(slot)
    engine.destroy()


@pytest.mark.parametrize("dtype,margin", [("float32", 1e-5), ("bfloat16", 6e-2)])
@pytest.mark.parametrize("name", ["mixed", "fast"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype, margin):
    """`Engine.generate` (the scheduler's batches, sampling on the device, one step ahead of the host): every token
    it chose is the plain logits' maximum, or within rounding of it."""
    raw = CONFIGS[name][0]
    prompts = [random_tokens(n, raw["vocab"], 60 + i) for i, n in enumerate((4, 150, 33, 71, 9))]
    engine = engine_for(folders[name], dtype, max_tokens=0, max_ctx=256)
    outs = engine.generate(prompts, max_new_tokens=12, temperature=0.0, stop_token_ids=[])
    for p, o in zip(prompts, outs):
        assert len(o.tokens) == 12
        ref = plain_logits(folders[name], p + o.tokens)
        for i, tok in enumerate(o.tokens):
            row = ref[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= margin * float(np.abs(row).max()), (i, tok, int(row.argmax()))
    engine.destroy()


def test_the_command_line_generates(folders, capsys):
    from odin_infer_b200 import cli
    assert cli.main([folders["odd"], "--prompt-ids", "1,2,3,4", "-n", "5", "-t", "0", "-c", "128", "--json"]) == 0
    out = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    assert out and len(out[0]["tokens"]) == 5


def random_config(seed: int) -> dict:
    """A configuration drawn at random: order and number of layers, every size, every constant."""
    rng = np.random.default_rng(seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]   # noqa: E731
    width = pick([40, 64, 72, 96, 100, 128])
    layers = []
    for _ in range(int(rng.integers(2, 7))):
        if rng.random() < 0.5:
            dim, rot = pick([8, 16, 24, 40, 64, 128]), pick([2, 8, 16, 32, 64])
            kv_rank = pick([16, 40, 64 - rot if rot < 64 else 64, 128 - rot, 96, 120])
            mx = latent(pick([1, 2, 3, 4, 8]), dim, rot, pick([dim, dim, 8, 48]), pick([12, 36, 64]), kv_rank,
                        pick([0, 1, 2, 17, 63, 64, 65, 130, 259]), float(rng.uniform(0.05, 0.3)), float(pick([1e3, 1e4, 1e6])))
            if rng.random() < 0.6:
                mx["rot"]["scaling"] = {"factor": float(pick([2, 8, 32])), "original": int(pick([32, 128, 2048])),
                                        "fast": float(pick([32, 8, 4])), "slow": float(pick([1, 0.5, 2]))}
            kind = "latent_attention"
        else:
            heads, dim = pick([1, 2, 3, 4, 6]), pick([8, 16, 24, 32, 64, 128])
            mx = retention(heads, dim, pick([dim, dim, 8, 48, 72]), [float(pick([0.5, 0.9, 0.97, 0.99, 0.999, 1.0])) for _ in range(heads)],
                           pick([0, dim, dim // 2, 2 * (dim // 8)]), float(pick([1e3, 1e4, 1e6])))
            kind = "retention"
        if rng.random() < 0.25:
            mlp = None
        else:
            groups = pick([1, 1, 2, 3, 4])
            per = pick([1, 2, 3, 4])
            keep = int(rng.integers(1, groups + 1))
            top = int(rng.integers(1, keep * per + 1))
            ff = pick([16, 40, 64])
            mlp = moe(groups * per, top, ff, None if (groups == 1 and rng.random() < 0.5) else (groups, keep),
                      None if rng.random() < 0.3 else float(rng.uniform(0.5, 3.0)), pick([0, ff, 2 * ff, ff + 8]))
        layers.append(layer(kind, mx, mlp))
    cfg = {"architecture": "Nikonex", "vocab": int(rng.integers(40, 400)), "width": width,
           "norm": {"eps": float(pick([1e-5, 1e-6]))}, "layers": layers}
    if rng.random() < 0.8:
        cfg["residual_mult"] = float(rng.uniform(0.3, 1.2))
    return cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [201, 202, 203, 204, 205, 206, 207, 208, 209, 210])
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    """Whole prompts, the last tokens one by one, and an unequal batch, for configurations that nobody chose."""
    raw = random_config(seed)
    folder = write_model(os.path.join(str(tmp_path), "m"), raw, seed)
    reqs = requests_for(raw, [1, 47, 290], seed=seed)
    engine = engine_for(folder, dtype)
    for recs in (traces.whole(reqs), traces.tail_one_by_one(reqs, tail=33), traces.batches(reqs, 3, first_part=lambda n: max(1, n - 20))):
        check_rows(traces.collect(recs, replay(engine, recs)), folder, reqs, dtype)
    engine.destroy()


# --------------------------------------------------------------------------------------
# every mechanism alone, with inputs that show a fault
# --------------------------------------------------------------------------------------
def close(got, ref, tol):
    got, ref = got.double().cpu(), ref.double().cpu()
    err = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert err <= tol, f"relative error {err:.3e} > {tol:.1e}"


def runtime(dtype):
    from odin_infer_b200.engine.runtime import Runtime
    return Runtime(DEV, dtype)


def cache_for(mixers, dtype, max_tokens=64 * 24, max_len=64 * 12):
    """A cache manager with storage and state for the given mixers (one schedule entry each)."""
    from odin_infer_b200.cache import CacheManager
    cache = CacheManager(max_tokens, max_len)
    for m in mixers:
        cache.add_entry(m.cache_request(), m.state_bytes())
    cache.entry_writes = [True] * len(mixers)
    for g in cache.groups.values():
        k = torch.full(g.storage_shape(), float("nan"), dtype=dtype, device=DEV)   # an unwritten row that is read shows
        g.attach_storage(k, k if g.request.shared_kv else torch.full(g.storage_shape(), float("nan"), dtype=dtype, device=DEV))
    cache.state = torch.full((cache.max_slots, max(cache.state_bytes_per_slot, 1)), 0x7f, dtype=torch.uint8, device=DEV)
    cache.zero_state = lambda slot: cache.state[slot].zero_()     # as the engine does when a slot is handed out
    return cache


def run_in_steps(mixer, rt, cache, h, cuts):
    """The mixer's output for one sequence whose rows h come in steps that end at the given cuts."""
    from odin_infer_b200.engine.step import StepBatch, StepEntry
    slot = cache.take_slot()
    outs, at = [], 0
    for end in cuts:
        st = cache.extend(slot, end - at)
        step = StepBatch(cache, [StepEntry(slot, [0] * (end - at), list(range(end - at)))], [st], DEV)
        o = mixer.forward(rt, step, h[at:end].contiguous(), 0)
        outs.append((o.sum(0) if o.dim() == 3 else o).float().clone())
        cache.after_step(slot)
        at = end
    cache.give_back_slot(slot)
    return torch.cat(outs)


def rope_part(rt, dims, base, scaling, layout, n):
    from odin_infer_b200.parts import PartSpec, build_part
    pe = build_part("position_encoding", PartSpec("rope", dict(rotary_dim=dims, theta=base, ramp=scaling, precise=True,
                                                               layout=layout, exact_angles=True)))
    pe.prepare(rt, n)
    return pe


LATENT_GEOMETRIES = [  # heads, dim, rot_dim, vdim, q_rank, kv_rank, window, tokens
    (3, 24, 8, 20, 36, 40, 37, 150),       # rows of 48: the CUDA-core kernels
    (4, 32, 64, 48, 40, 64, 64, 200),      # rows of 128, a window of exactly a page
    (2, 16, 16, 24, 24, 48, 65, 200),      # rows of 64, a window of a page and a key
    (8, 16, 32, 16, 32, 96, 130, 330),     # rows of 128, a window over three pages
    (2, 40, 6, 8, 16, 50, 1, 70),          # a window of the query's own key
    (1, 8, 32, 8, 8, 32, 0, 140),          # no window
    (20, 8, 16, 8, 24, 112, 100, 260)]     # more heads than a tensor-core tile of queries takes


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("geom", LATENT_GEOMETRIES)
def test_latent_attention_alone_with_loud_keys_at_the_windows_edge(dtype, tol, geom):
    """A few tokens are thirty times louder than the rest: the key/value latent is normed and does not care, the
    rotated key part is not, so their scores (positive for some heads and queries, negative for others) dwarf all
    others.  A query sees such a token up to `window - 1` tokens later and not one more: whole prompt, portions that
    end around the loud tokens and around the pages' borders, and the last sixty tokens one by one."""
    from odin_infer_b200.parts import PartSpec, build_part
    H, e, r, ev, qr, kvr, window, n = geom
    width = 72
    rt = runtime(dtype)
    names = {k: "m." + v for k, v in dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", o="o").items()}
    scaling = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    att = build_part("mixer", PartSpec("latent_attention", dict(
        width=width, n_heads=H, head_dim=e, rot_dim=r, v_head_dim=ev, q_rank=qr, kv_rank=kvr, names=names,
        position_encoding="pe", eps=1e-5, scale=0.17, window=window)))
    att.pe = rope_part(rt, r, 3000.0, scaling, "pairs", n)
    torch.manual_seed(H * 1000 + window)
    t = {p.name: torch.randn(p.shape, device=DEV) / math.sqrt(p.shape[-1]) if len(p.shape) == 2
         else 1.0 + 0.2 * torch.randn(p.shape, device=DEV) for p in att.params()}
    t = {k: v.to(dtype) for k, v in t.items()}
    ref_w = {k: v.double().cpu() for k, v in t.items()}
    att.bind(dict(t), rt)
    h = torch.randn(n, width, device=DEV)
    loud = sorted({5, 63, 64, n - 61, n - 1 - max(window, 1), n - max(window, 1)} & set(range(n)))
    h[loud] *= 30.0
    h = h.to(dtype)
    mx = {"heads": H, "dim": e, "rot_dim": r, "vdim": ev, "q_rank": qr, "kv_rank": kvr, "scale": 0.17,
          "rot": {"dims": r, "base": 3000.0, "scaling": scaling}}
    if window:
        mx["mask"] = {"size": window}
    ref = P.latent_attention(h.double().cpu(), ref_w, "m.", mx, 1e-5)
    if dtype == torch.bfloat16:
        # scores of loud keys are large, and so is what bfloat16 takes off them: the limit is three times what
        # rounding of the stored activations alone does here, where that is more than the tolerance
        noisy = P.latent_attention(h.double().cpu(), ref_w, "m.", mx, 1e-5, rnd=P.to_bfloat16_and_back)
        tol = max(tol, 3.0 * float((noisy - ref).abs().max() / ref.abs().max()))
    cache = cache_for([att], dtype)
    for cuts in ([n], sorted({3, 64, 66, 128, n - 2, n} & set(range(1, n + 1))), list(range(n - 60, n + 1))):
        got = run_in_steps(att, rt, cache, h, cuts)
        close(got, ref, tol)
    if window and n - window - 1 >= 0:
        # the same with a window that is one key longer is far off: the edge is no rounding matter
        mx2 = dict(mx, mask={"size": window + 1})
        other = P.latent_attention(h.double().cpu(), ref_w, "m.", mx2, 1e-5)
        assert (other - ref).abs().max() > 0.25 * ref.abs().max()
    cache.check()


RETENTION_GEOMETRIES = [  # heads, dim, vdim, decays, rot dims, layout, tokens
    (2, 24, 40, [0.9, 0.9995], 16, "halves", 300),
    (3, 16, 16, [0.5, 1.0, 0.0], 16, "halves", 150),
    (1, 64, 64, [0.999], 32, "halves", 400),
    (4, 32, 8, [0.97, 0.98, 0.99, 0.995], 0, "halves", 130),
    (2, 128, 72, [0.99, 0.95], 128, "pairs", 200)]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("geom", RETENTION_GEOMETRIES)
def test_retention_alone_remembers_a_loud_token_far_back(dtype, tol, geom):
    """Token 7 is thirty times louder than the rest (its key and its value both): a head with a decay near one still
    hears it hundreds of tokens later, a head with a small decay has forgotten it, and a state that is lost or reset
    between steps loses it for all.  Whole, in portions down to two tokens, and the last forty tokens one by one."""
    from odin_infer_b200.parts import PartSpec, build_part
    H, e, ev, decay, rot, layout, n = geom
    width = 80
    rt = runtime(dtype)
    ret = build_part("mixer", PartSpec("retention", dict(width=width, n_heads=H, head_dim=e, v_head_dim=ev, decay=decay,
                                                         names={k: "m." + k for k in "qkvgo"},
                                                         position_encoding="pe" if rot else None, eps=1e-5)))
    if rot:
        ret.pe = rope_part(rt, rot, 700.0, None, layout, n)
    torch.manual_seed(H * 100 + e)
    t = {p.name: (torch.randn(p.shape, device=DEV) / math.sqrt(p.shape[-1])).to(dtype) for p in ret.params()}
    ref_w = {k: v.double().cpu() for k, v in t.items()}
    ret.bind(dict(t), rt)
    h = torch.randn(n, width, device=DEV)
    h[7] *= 30.0
    h = h.to(dtype)
    mx = {"heads": H, "dim": e, "vdim": ev, "decay": decay}
    if rot:
        mx["rot"] = {"dims": rot, "base": 700.0}
    if layout == "pairs":      # the part takes either layout; the plain mixer turns halves: compare through its pieces
        ref = _plain_retention_in_pairs(h.double().cpu(), ref_w, mx)
    else:
        ref = P.retention(h.double().cpu(), ref_w, "m.", mx, 1e-5)
    # the loud token matters at the end for the slow head: without it the last row is another row
    quiet = h.clone()
    quiet[7] /= 30.0
    if max(decay) >= 0.99 and layout == "halves":
        other = P.retention(quiet.double().cpu(), ref_w, "m.", mx, 1e-5)
        assert (other[-1] - ref[-1]).abs().max() > 0.25 * ref[-1].abs().max()
    cache = cache_for([ret], dtype)
    for cuts in ([n], [2, 4, 7, 8, 64, 65, n - 3, n], list(range(n - 40, n + 1))):
        close(run_in_steps(ret, rt, cache, h, cuts), ref, tol)
    # the slot's state is cleared when the next sequence takes it
    close(run_in_steps(ret, rt, cache, quiet, [n])[-1], P.retention(quiet.double().cpu(), ref_w, "m.", mx, 1e-5)[-1]
          if layout == "halves" else _plain_retention_in_pairs(quiet.double().cpu(), ref_w, mx)[-1], tol)


def _plain_retention_in_pairs(h, w, mx):
    n, H, e, ev = h.shape[0], mx["heads"], mx["dim"], mx["vdim"]
    freqs, _ = P.ramp_frequencies(mx["rot"]["dims"], mx["rot"]["base"], None)
    q = P.rotate((h @ w["m.q"].T).view(n, H, e), range(n), freqs, 1.0, "pairs")
    k = P.rotate((h @ w["m.k"].T).view(n, H, e), range(n), freqs, 1.0, "pairs") * float(e) ** -0.5
    v = (h @ w["m.v"].T).view(n, H, ev)
    o = torch.zeros(n, H, ev, dtype=F64)
    for hd in range(H):
        S = torch.zeros(e, ev, dtype=F64)
        for t in range(n):
            S = mx["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    g = h @ w["m.g"].T
    return (P.rms(o, None, 1e-5).reshape(n, H * ev) * g * torch.sigmoid(g)) @ w["m.o"].T


@pytest.mark.parametrize("E,groups,keep,top", [(6, 3, 2, 2), (16, 4, 1, 4), (8, 8, 3, 3), (12, 1, 1, 5), (32, 2, 2, 32), (9, 3, 3, 1), (64, 32, 5, 7)])
@pytest.mark.parametrize("given_logits", [False, True])
def test_router_in_groups(E, groups, keep, top, given_logits):
    """Choices and weights against the plain router, with scores that are distinct by construction (no close calls);
    groups of one expert, all groups kept, one group; the logits formed here or handed in; padding rows; the gate row."""
    from odin_infer_b200.csrc import ops
    torch.manual_seed(E + groups)
    T, d = 11, 40
    h = torch.randn(T, d, device=DEV)
    w = torch.randn(E + 1, d, device=DEV) * 2 / math.sqrt(d)
    tok_seq = torch.tensor([0, 0, 1, -1, 2, 2, 2, -1, 3, 3, 4], dtype=torch.int32, device=DEV)
    ids = torch.empty(T, top + 2, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top + 2, dtype=torch.float32, device=DEV)
    gate = torch.empty(T, dtype=torch.float32, device=DEV)
    logits = (h @ w.T).contiguous() if given_logits else None
    ops.moe_router(h, w, None, top, 2, tok_seq, ids, wts, logits, score="sigmoid_in_groups", groups=groups, keep=keep,
                   route_scale=1.7, gate_row=True, gate_out=gate)
    router = {"experts": E, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}
    ref_ids, ref_w = P.route(h.double().cpu(), w[:E].double().cpu(), router)
    real = (tok_seq >= 0).cpu()
    want_gate = torch.sigmoid(h.double().cpu() @ w[E].double().cpu())
    for t in range(T):
        if not real[t]:
            assert (ids[t].cpu() == -1).all() and (wts[t].cpu() == 0).all() and float(gate[t]) == 0.0
            continue
        assert ids[t, :top].cpu().tolist() == ref_ids[t], (t, ids[t].cpu().tolist(), ref_ids[t])
        close(wts[t, :top], ref_w[t], 1e-5)
        assert ids[t, top:].cpu().tolist() == [E, E + 1]
        close(wts[t, top:], want_gate[t].expand(2), 1e-5)
        close(gate[t], want_gate[t], 1e-5)


def test_ties_in_groups_go_to_the_lower_index():
    from odin_infer_b200.csrc import ops
    h = torch.ones(2, 8, device=DEV)
    w = torch.zeros(6, 8, device=DEV)
    ids = torch.empty(2, 2, dtype=torch.int32, device=DEV)
    wts = torch.empty(2, 2, dtype=torch.float32, device=DEV)
    ops.moe_router(h, w, None, 2, 0, None, ids, wts, None, score="sigmoid_in_groups", groups=3, keep=1, route_scale=3.0)
    assert ids.cpu().tolist() == [[0, 1], [0, 1]] and torch.allclose(wts.cpu(), torch.full((2, 2), 1.5))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2.5e-2)])
@pytest.mark.parametrize("T", [7, 200])
@pytest.mark.parametrize("E,groups,keep,top,ff,shared", [(6, 3, 2, 2, 40, 56), (8, 2, 1, 3, 32, 64), (4, 1, 1, 4, 24, 0), (5, 5, 2, 1, 16, 16)])
def test_feed_forward_of_experts_with_a_gated_shared_expert(dtype, tol, T, E, groups, keep, top, ff, shared):
    """The whole feed-forward part against the plain one: few rows (row-by-row kernels) and many (grouped tensor-core
    products); a shared expert of the experts' size or twice (rides with them, its gate as their weight), of another
    size (runs beside them, its gate on the activations), and none.  The router's rows are spread so that rounding of
    what it reads cannot change a choice."""
    from odin_infer_b200.parts import PartSpec, build_part
    width = 64
    rt = runtime(dtype)
    names = {"router": "f.router", "up": "f.e{e}.up", "down": "f.e{e}.down", "shared_up": "f.shared.up",
             "shared_down": "f.shared.down", "shared_token_gate": "f.shared.sg"}
    ffn = build_part("feed_forward", PartSpec("routed_experts", dict(
        width=width, inner=ff, n_experts=E, top=top, activation="relu2", gated=False, shared_inner=shared,
        score="sigmoid_in_groups", groups=groups, keep=keep, route_scale=2.2, shared_gate=shared > 0, names=names)))
    torch.manual_seed(E * 10 + T)
    t = {}
    for p in ffn.params():
        r = torch.randn(p.shape, device=DEV)
        t[p.name] = (r * (6.0 if p.name.endswith(("router", ".sg")) else 1.0) / math.sqrt(p.shape[-1])).to(dtype)
    ref_w = {k: v.double().cpu() for k, v in t.items()}
    ffn.bind(dict(t), rt)
    h = torch.randn(T, width, device=DEV).to(dtype)

    class Step:
        tok_seq = None
    out = ffn.forward(rt, Step(), h)
    parts = list(out) if isinstance(out, list) else [out]
    total = sum((o.float().sum(0) if o.dim() == 3 else o.float()) for o in parts)
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "top": top, "scale": 2.2, "groups": {"count": groups, "keep": keep}}}
    if shared:
        mlp["shared"] = {"ff": shared}
    want = P.expert_mlp(h.double().cpu(), ref_w, "f.", mlp)
    if dtype == torch.float32:
        close(total, want, tol)
    else:
        # rows whose choice was a close call for bfloat16 inputs may differ by an expert: nine rows in ten must not
        err = (total.double().cpu() - want).abs().amax(dim=1) / want.abs().max()
        assert (err > tol).sum() <= max(1, T // 10) and err.median() <= tol / 4, (int((err > tol).sum()), float(err.max()))


@pytest.mark.parametrize("pairs", [True, False])
def test_rotation_of_heads_in_both_layouts(pairs):
    """The rotation kernel against the plain rotation: partial rotation, the factor from a head on, in place and
    into a wider row, positions far along the table, a gain on cos and sin."""
    from odin_infer_b200.csrc import ops
    rt = runtime(torch.float32)
    layout = "pairs" if pairs else "halves"
    scaling = {"factor": 8.0, "original": 40, "fast": 4.0, "slow": 0.5}
    pe = rope_part(rt, 12, 500.0, scaling, layout, 700)
    cos, sin, rot = pe.rotation()
    assert rot == 12
    T, H, width = 9, 5, 20
    torch.manual_seed(3)
    src = torch.randn(T, H * width, device=DEV)
    pos = torch.tensor([0, 1, 2, 63, 64, 65, 300, 698, 699], dtype=torch.int32, device=DEV)
    dst = torch.zeros(T, H * (width + 4), device=DEV)
    ops.rope_heads(src, width, dst[:, 4:], width + 4, H, width, rot, pairs, cos, sin, pos, scale=0.25, scale_from_head=3)
    freqs, gain = P.ramp_frequencies(12, 500.0, scaling)
    want = P.rotate(src.double().cpu().view(T, H, width), pos.cpu().tolist(), freqs, gain, layout)
    want[:, 3:] *= 0.25
    got = dst.view(T, H, width + 4)
    # a 32-bit angle of a few hundred radians is good to about 1e-5
    close(got[:, :, 4:], want, 1e-4)
    assert (got[:, 1:, :4] == 0).all()
    same = src.clone()
    ops.rope_heads(same, width, same, width, H, width, rot, pairs, cos, sin, pos, scale=0.25, scale_from_head=3)
    close(same.view(T, H, width), want, 1e-4)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 8e-3)])
def test_a_product_per_head_and_the_unit_norm_with_its_gate(dtype, tol):
    from odin_infer_b200.csrc import ops
    torch.manual_seed(4)
    T, H, K, N = 19, 3, 37, 50
    a = torch.randn(T, H * (K + 5), device=DEV).to(dtype)
    w = (torch.randn(H, K, N, device=DEV) / math.sqrt(K)).to(dtype)
    out = torch.zeros(T, H * N, dtype=dtype, device=DEV)
    ops.heads_linear(a, K + 5, w, out, N)
    want = torch.einsum("thk,hkn->thn", a.double().cpu().view(T, H, K + 5)[:, :, :K], w.double().cpu())
    close(out.view(T, H, N), want, tol)
    o = torch.randn(T, H * N, device=DEV) * torch.tensor([1e-3, 1.0, 50.0], device=DEV).repeat_interleave(N)
    g = torch.randn(T, H * N, device=DEV)
    y = torch.empty(T, H * N, dtype=dtype, device=DEV)
    ops.head_unit_scale(o, None, False, g, 1e-5, y, H, N)
    gd = g.double().cpu()
    want = P.rms(o.double().cpu().view(T, H, N), None, 1e-5).reshape(T, H * N) * gd * torch.sigmoid(gd)
    close(y, want, tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("T,H,K,N", [(200, 3, 37, 50), (64, 2, 64, 64), (33, 1, 130, 7), (321, 5, 8, 96)])
def test_a_product_per_head_of_many_tokens_has_the_bits_of_few(dtype, tol, T, H, K, N):
    """Many tokens go through tiles in shared memory, few through a kernel of their own: the same sums in the same order,
    so a token's values do not depend on how many others come with it; and against float64, into a strided output."""
    from odin_infer_b200.csrc import ops
    torch.manual_seed(T + K)
    a = torch.randn(T, H * (K + 3), device=DEV).to(dtype)
    w = (torch.randn(H, K, N, device=DEV) / math.sqrt(K)).to(dtype)
    out = torch.full((T, H * (N + 2)), 5.0, dtype=dtype, device=DEV)
    ops.heads_linear(a, K + 3, w, out, N + 2)
    want = torch.einsum("thk,hkn->thn", a.double().cpu().view(T, H, K + 3)[:, :, :K], w.double().cpu())
    got = out.view(T, H, N + 2)
    close(got[:, :, :N], want, tol)
    assert (got[:, :, N:] == 5.0).all()   # what lies between the heads' outputs is left alone
    few = torch.full_like(out, 5.0)
    for t0 in range(0, T, 9):
        ops.heads_linear(a[t0:t0 + 9], K + 3, w, few[t0:t0 + 9], N + 2)
    assert torch.equal(out, few)


@pytest.mark.parametrize("act", ["relu2", "silu", "gelu_tanh"])
@pytest.mark.parametrize("E,K,N", [(3, 64, 40), (5, 72, 152), (2, 128, 256)])
def test_grouped_product_without_a_gate_applies_its_activation_as_it_reads_back(act, E, K, N):
    """Sorted rows times their tile's own expert on the tensor cores, act(a W^T) written in bfloat16: against a loop in
    float64, over an expert without a tile, an output that is no multiple of the tile and a K that is no multiple of 64."""
    from odin_infer_b200.csrc import ops
    torch.manual_seed(E * K + N)
    tiles = [0, E - 1, -1, 0] if E > 2 else [1, -1, 1]
    tile_expert = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    places = 128 * len(tiles)
    a = torch.randn(places, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(E, N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    out = torch.full((places, N), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.moe_grouped(a, w, tile_expert, out, act, gated=False)
    torch.cuda.synchronize()
    ops.moe_tc_check()
    f = {"relu2": lambda z: z.clamp(min=0) ** 2, "silu": lambda z: z * torch.sigmoid(z),
         "gelu_tanh": lambda z: 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}[act]
    for i, e in enumerate(tiles):
        rows = slice(128 * i, 128 * (i + 1))
        if e < 0:
            assert (out[rows] == 7.0).all()   # a tile that no expert's rows reach is left alone
            continue
        want = f(a[rows].double().cpu() @ w[e].double().cpu().T)
        close(out[rows], want, 8e-3)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("d,groups,scale,updates", [(96, 1, 0.37, 2), (130, 2, 1.0, 1), (200, 1, 1.0, 0), (64, 4, 2.5, 3)])
def test_two_norms_of_one_updated_row(out_dtype, d, groups, scale, updates):
    """x += scale * (sum of the updates), then two norms of that one row with weights of their own from one root mean
    square: against float64, with and without updates, in groups, at a width that is no multiple of four, and through
    a gather of rows (which leaves x as it was)."""
    from odin_infer_b200.csrc import ops
    torch.manual_seed(d + updates)
    n = 37
    x0 = torch.randn(n, d, device=DEV) * 3
    first = torch.randn(n, d, device=DEV).to(out_dtype) if updates else None
    rest = [torch.randn(2, n, d, device=DEV) if i == 0 else torch.randn(n, d, device=DEV) for i in range(max(updates - 1, 0))]
    w1, w2 = torch.rand(d, device=DEV) + 0.5, torch.randn(d, device=DEV)
    x = x0.clone()
    o1, o2 = torch.empty(n, d, dtype=out_dtype, device=DEV), torch.full((n, d), 9.0, dtype=out_dtype, device=DEV)
    delta = None if first is None else ([first] + rest if rest else first)
    ops.row_update(x, delta, None, w1, 1e-5, groups, o1, scale=scale if updates else 1.0, weight2=w2, out2=o2)
    torch.cuda.synchronize()
    total = torch.zeros(n, d, dtype=torch.float64)
    if first is not None:
        total += first.double().cpu()
    for m in rest:
        total += m.double().cpu().reshape(-1, n, d).sum(0)
    want_x = x0.double().cpu() + scale * total
    close(x, want_x, 1e-6)
    parts = want_x.view(n, groups, d // groups)
    unit = (parts / torch.sqrt((parts ** 2).mean(-1, keepdim=True) + 1e-5)).reshape(n, d)
    tol = 1e-5 if out_dtype == torch.float32 else 8e-3
    close(o1, unit * w1.double().cpu(), tol)
    close(o2, unit * w2.double().cpu(), tol)
    rows = torch.tensor([5, -1, 0, 36], dtype=torch.int32, device=DEV)
    p1, p2 = torch.empty(4, d, dtype=out_dtype, device=DEV), torch.empty(4, d, dtype=out_dtype, device=DEV)
    kept = x.clone()
    ops.row_update(x, None, None, w1, 1e-5, groups, p1, rows, weight2=w2, out2=p2)
    torch.cuda.synchronize()
    assert torch.equal(x, kept)
    pick = torch.tensor([5, 0, 36])
    assert torch.equal(p1[[0, 2, 3]], o1[pick.to(DEV)]) and torch.equal(p2[[0, 2, 3]], o2[pick.to(DEV)])
    assert (p1[1] == 0).all() and (p2[1] == 0).all()
