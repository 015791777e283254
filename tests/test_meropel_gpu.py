"""The Meropel decoder through the engine against its plain implementation (tests/plain/meropel_plain.py):
every mechanism alone, whole prompts against token-by-token decoding, prompts in portions, unequal batches,
slots, pages and states that are used again, the first tokens of a sequence, long decoding, sizes that the fast
kernels take and sizes that they do not, and greedy generation through the engine's own entry point.  The tests
write their own weights and inputs (matrices of unit gain, decays that remember for hundreds of tokens, a router
whose scores spread and whose correction changes the choice, a loud key far back) so that a lost state, a forgotten
token before, a group that is scored wrongly or a pair that is rotated in the wrong layout leaves a mark far above
rounding."""
import json
import math
import os

import numpy as np
import pytest
import torch

from tests import traces
from tests.plain import meropel_plain as P
from tests.tiny import TOL, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def attn(heads, kv, dim, vdim, scale, rot=0, base=1e4):
    out = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        out["rot"] = {"dims": rot, "base": base}
    return out


def par(left, inner, state, rank, conv, ls, rs):
    return {"left": left, "left_scale": ls, "right": {"inner": inner, "state": state, "dt_rank": rank, "conv": conv},
            "right_scale": rs}


def par2(left, heads, vdim, state, groups, norm_groups, conv):
    return {"left": left, "right": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                    "norm_groups": norm_groups, "conv": conv}}


def moe(experts, identity, top, ff, count=1, keep=1, scale=1.0, shared=0):
    out = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "top": top, "scale": scale, "identity": identity,
                      "groups": {"count": count, "keep": keep}}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(kind, mx, mlp):
    return {"type": kind, "mixer": mx, "mlp": mlp}


BIGRAM = {"bigram": {"buckets": 61, "mul_prev": 31, "mul_cur": 5}}

# odd sizes throughout; value heads larger and smaller than keys; partial and no rotation; a shared expert that rides with the
# experts (twice their size) and one that runs beside them; pass-through rows in two layers; a layer without feed-forward
MIXED = {"architecture": "Meropel", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.7, "embedding": BIGRAM,
         "layers": [layer("parallel", par(attn(4, 2, 24, 40, 0.3, rot=8), 72, 12, 5, 3, 0.7, 1.3), {"kind": "dense", "ff": 80}),
                    layer("gla", {"heads": 3, "dim": 20, "vdim": 28, "tau": 8.0}, moe(6, 3, 3, 40, 3, 2, 2.0, shared=80)),
                    layer("parallel_2", par2(attn(4, 1, 32, 32, 0.2, rot=32, base=5e5), 4, 16, 24, 2, 4, 4), None),
                    layer("parallel", par(attn(2, 2, 16, 8, 0.25), 40, 5, 3, 2, 1.0, 0.4), moe(5, 1, 2, 24, 2, 2, 1.0, shared=56))]}
# a width that is no multiple of 8; one head, one group, one expert per token, every router row chosen, a convolution of one tap
ODD = {"architecture": "Meropel", "vocab": 97, "width": 100, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
       "embedding": {"bigram": {"buckets": 7, "mul_prev": 1, "mul_cur": 1}},
       "layers": [layer("parallel_2", par2(attn(3, 3, 20, 28, 0.22, rot=12, base=300.0), 1, 36, 9, 1, 1, 1), moe(4, 0, 1, 20)),
                  layer("gla", {"heads": 1, "dim": 36, "vdim": 12, "tau": 1.0}, moe(3, 1, 4, 16, 4, 4, 0.5)),
                  layer("parallel", par(attn(5, 1, 12, 20, 0.29, rot=12, base=50.0), 52, 40, 1, 5, 1.0, 1.0), None)]}
# head sizes the tensor-core attention kernels take, widths the tensor-core products take
FAST = {"architecture": "Meropel", "vocab": 512, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 0.5, "embedding": BIGRAM,
        "layers": [layer("parallel", par(attn(4, 2, 64, 64, 0.11, rot=32), 256, 16, 8, 4, 0.9, 0.6), moe(7, 3, 2, 64, 5, 3, 1.25, shared=64)),
                   layer("parallel_2", par2(attn(2, 1, 128, 128, 0.09, rot=64, base=1e6), 8, 32, 64, 2, 2, 4), {"kind": "dense", "ff": 256}),
                   layer("gla", {"heads": 2, "dim": 64, "vdim": 128, "tau": 12.0}, moe(16, 0, 4, 64, 4, 2, 1.0))]}
CONFIGS = {"mixed": (MIXED, 3), "odd": (ODD, 5), "fast": (FAST, 7)}


def make_weight(name: str, shape, gen) -> torch.Tensor:
    """Weights of the tests' own making: matrices N(0, 1/in), norm weights around one, a router of gain 3 with a
    correction of the scores' own size, step sizes and decays that remember for tens to hundreds of tokens."""
    r = torch.randn(shape, generator=gen)
    last = name.rsplit(".", 1)[-1]
    if name.endswith((".q.norm", ".k.norm")) or last in ("norm1", "norm2", "norm1b", "norm2b", "norm", "out", "D"):
        return 1.0 + 0.3 * r
    if name in ("embed", "bigram"):
        return r
    if last == "router":
        return 3.0 * r / math.sqrt(shape[1])
    if last == "correction":
        return 0.1 * r
    if name.endswith(("conv.b", ".q.b", ".k.b", ".v.b")):
        return 0.3 * r
    if last == "conv":
        return 0.6 * r
    if name.endswith(("dt.b", "dt_bias")):
        return -2.5 + 1.2 * r
    if last == "A_log":
        return -0.5 + 0.8 * r
    if name.endswith("a2.b"):
        return 2.0 + 1.5 * r
    if last == "dt" and len(shape) == 2:
        return r / math.sqrt(shape[1])
    if last in ("o", "down"):
        return 0.5 * r / math.sqrt(shape[1])
    return r / math.sqrt(shape[-1])


def write_model(folder: str, raw: dict, seed: int) -> str:
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.weights import model_param_specs
    from odin_infer_b200.weights.safetensors_io import write_safetensors
    cfg = config_from_dict(raw)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    gen = torch.Generator().manual_seed(seed)
    specs = model_param_specs(cfg)
    shapes = {s.name: s.concrete_shape for s in specs}
    write_safetensors(os.path.join(folder, "model.safetensors"), [(s.name, torch.bfloat16, s.concrete_shape) for s in specs],
                      lambda name: make_weight(name, shapes[name], gen).to(torch.bfloat16))
    return folder


_folders = {}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    if not _folders:
        base = tmp_path_factory.mktemp("meropel")
        for name, (raw, seed) in CONFIGS.items():
            _folders[name] = write_model(os.path.join(str(base), name), raw, seed)
    return _folders


_plain = {}


def plain_logits(folder, tokens, rounded=None):
    """rounded: None (exact), "bfloat16" or "float32": what an engine of that type stores between kernels is rounded to it."""
    key = (folder, tuple(tokens), rounded)
    if key not in _plain:
        cfg, w = P.read_model_folder(folder, F64)
        rnd = {None: lambda t: t, "bfloat16": P.to_bfloat16_and_back, "float32": lambda t: t.float().double()}[rounded]
        _plain[key] = P.forward(cfg, w, tokens, rnd=rnd).numpy()
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


# The 32-bit engine is held to the tolerance at every position, or to five times what rounding to 32 bits alone does
# there where that is more (a head's norm of an output that nearly cancels amplifies the last bits: at a sequence's
# first position a linear-attention head's output is (q . k) v, and its norm turns on the sign of a small q . k).
# In bfloat16 the yardstick is what rounding alone does
# to this model and these tokens (the plain implementation run again with what a 16-bit engine stores rounded to
# bfloat16): a router's close call that falls the other way changes a token's update by an expert's share, and the
# recurrent layers carry that on, so a position's limit is the tolerance or three times the rounding's own error there,
# one position in ten may be over it, and the median stays within twice the rounding's median.
def check_rows(got: dict, folder, requests, dtype):
    for rid, rows in got.items():
        n = rows.shape[0]
        ref = plain_logits(folder, requests[rid])[:n]
        top = max(np.abs(ref).max(), 1e-30)
        err = np.abs(rows.astype(np.float64) - ref).max(axis=1) / top
        if dtype == "float32":
            if err.max() > TOL[dtype]:
                noise = np.abs(plain_logits(folder, requests[rid], rounded="float32")[:n] - ref).max(axis=1) / top
                worst = int((err / np.maximum(TOL[dtype], 5.0 * noise)).argmax())
                assert (err <= np.maximum(TOL[dtype], 5.0 * noise)).all(), \
                    f"{rid}: relative error {err[worst]:.3e} at {worst} (rounding to 32 bits alone {noise[worst]:.3e})"
            continue
        noise = np.abs(plain_logits(folder, requests[rid], rounded="bfloat16")[:n] - ref).max(axis=1) / top
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
    """Whole prompts (across several pages), then the same with the last tokens one by one, so that the recurrent
    states, the convolutions' last inputs and the token before pass from the prompt's kernels to the single-token ones;
    the first tokens of a sequence alone (prompts of 1 and 2)."""
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
                                        ("mixed", (2,)), ("odd", (1, 3))])
def test_prompts_in_portions(folders, name, sizes, dtype):
    """Portions of several sizes, down to two tokens and one: a portion starts from the states, the convolutions' last
    inputs (also when the portion is shorter than the convolution) and the token before that the portion before it left."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [150, 41] if len(sizes) <= 2 else [333, 77], seed=10)
    engine = engine_for(folders[name], dtype)
    recs = portions(reqs, sizes)
    check_rows(traces.collect(recs, replay(engine, recs)), folders[name], reqs, dtype)
    engine.destroy()


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batches_and_reuse(folders, name, dtype, graphs):
    """Batches of unequal requests, batch after batch in a cache that holds one batch only, so that every slot, every
    page and every slot's state is used again (a state, a convolution's memory or a token before that is not cleared
    shows in the next request); shorter requests end earlier."""
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
    """In 32-bit a position's logits agree to rounding whole, in portions, one by one and in a batch, and a batch is the
    same bits as each request alone in the same cut."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [140, 59], seed=40)
    engine = engine_for(folders[name], "float32")
    ref = traces.collect(traces.whole(reqs), replay(engine, traces.whole(reqs)))
    for recs in (portions(reqs, (3, 50, 2)), traces.tail_one_by_one(reqs, tail=25), traces.batches(reqs, 2)):
        got = traces.collect(recs, replay(engine, recs))
        for rid in reqs:
            top = np.abs(ref[rid]).max()
            assert np.abs(got[rid] - ref[rid]).max() <= 4e-6 * top, rid
    alone = traces.collect(traces.batches(reqs, 1), replay(engine, traces.batches(reqs, 1)))
    both = traces.collect(traces.batches(reqs, 2), replay(engine, traces.batches(reqs, 2)))
    for rid in reqs:
        assert np.array_equal(alone[rid], both[rid]), rid
    engine.destroy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "fast"])
def test_long_decoding(folders, name, dtype):
    """Three hundred tokens decoded one by one after a short prompt: every state is carried three hundred times, the
    keys grow over page borders."""
    raw = CONFIGS[name][0]
    reqs = requests_for(raw, [330, 318], seed=50)
    recs = traces.batches(reqs, 2, first_part=lambda n: 12)
    engine = engine_for(folders[name], dtype)
    check_rows(traces.collect(recs, replay(engine, recs)), folders[name], reqs, dtype)
    assert all(g.pool.n_held == 0 for g in engine.cache.groups.values())
    engine.destroy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt(folders, dtype):
    """A prompt of 1,100 tokens whole, and with its last 40 tokens one by one: recurrences over many blocks of tokens,
    experts with several tiles of rows each, keys many pages back."""
    raw = CONFIGS["fast"][0]
    reqs = requests_for(raw, [1100], seed=70)
    engine = engine_for(folders["fast"], dtype, max_tokens=2048, max_ctx=1280)
    for recs in (traces.whole(reqs), traces.tail_one_by_one(reqs, tail=40)):
        check_rows(traces.collect(recs, replay(engine, recs)), folders["fast"], reqs, dtype)
    engine.cache.check()
    engine.destroy()


def test_what_a_sequence_holds(folders):
    """Attention branches with equal heads share a group of the cache; the state area holds, per sequence, every
    recurrent layer's state, its convolution's last inputs, and the token before."""
    engine = engine_for(folders["mixed"], "float32")
    shapes = sorted((g.request.n_kv_heads, g.request.head_dim, g.request.value_dim, g.n_lines) for g in engine.cache.groups.values())
    assert shapes == [(1, 32, 32, 1), (2, 16, 8, 1), (2, 24, 40, 1)], shapes
    want = [4 * (72 * 12 + 2 * 72), 4 * 3 * 20 * 28, 4 * (4 * 24 * 16 + 3 * (64 + 2 * 2 * 24)), 4 * (40 * 5 + 1 * 40), 4]
    assert engine.cache.state_bytes_of == want, engine.cache.state_bytes_of
    engine.destroy()


@pytest.mark.parametrize("dtype,margin", [("float32", 1e-5), ("bfloat16", 6e-2)])
@pytest.mark.parametrize("name", ["mixed", "fast"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype, margin):
    """`Engine.generate` (the scheduler's batches, sampling on the device, one step ahead of the host, so that the token
    before is taken from the device too): every token it chose is the plain logits' maximum, or within rounding of it."""
    raw = CONFIGS[name][0]
    prompts = [random_tokens(n, raw["vocab"], 60 + i) for i, n in enumerate((4, 150, 33, 71, 9))]
    engine = engine_for(folders[name], dtype, max_tokens=0, max_ctx=256)
    outs = engine.generate(prompts, max_new_tokens=12, temperature=0.0, stop_token_ids=[])
    off = []
    for p, o in zip(prompts, outs):
        assert len(o.tokens) == 12
        ref = plain_logits(folders[name], p + o.tokens)
        for i, tok in enumerate(o.tokens):
            row = ref[len(p) - 1 + i]
            if float(row.max() - row[tok]) > margin * float(np.abs(row).max()):
                off.append((i, tok, int(row.argmax())))
    # in bfloat16 a router's close call may fall the other way for a token (an expert's share of its update differs): two of
    # the sixty tokens may lie outside the margin; in 32-bit none
    assert len(off) <= (2 if dtype == "bfloat16" else 0), off
    engine.destroy()


def test_the_command_line_generates(folders, capsys):
    from odin_infer_b200 import cli
    assert cli.main([folders["odd"], "--prompt-ids", "1,2,3,4", "-n", "5", "-t", "0", "-c", "128", "--json"]) == 0
    out = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    assert out and len(out[0]["tokens"]) == 5


def random_config(seed: int) -> dict:
    rng = np.random.default_rng(seed)

    def pick(*xs):
        return xs[int(rng.integers(len(xs)))]

    def attention():
        kv = pick(1, 2, 3)
        dim = pick(8, 16, 24, 64)
        return attn(kv * pick(1, 2, 3), kv, dim, pick(8, 16, 40, dim), float(rng.uniform(0.1, 0.4)),
                    rot=pick(0, 4, dim // 2, dim), base=pick(100.0, 1e4, 1e6))

    def mlp():
        kind = pick(None, "dense", "moe", "moe")
        if kind is None:
            return None
        if kind == "dense":
            return {"kind": "dense", "ff": pick(24, 40, 64)}
        count = pick(1, 2, 3)
        size = pick(1, 2, 4)
        rows = count * size
        ident = int(rng.integers(0, max(1, rows // 2) + 1)) if rows > 1 else 0
        keep = int(rng.integers(1, count + 1))
        top = int(rng.integers(1, keep * size + 1))
        ff = pick(16, 24, 32)
        return moe(rows - ident, ident, top, ff, count, keep, float(rng.uniform(0.5, 2.5)), shared=pick(0, ff, 2 * ff, 40))

    layers = []
    for _ in range(int(rng.integers(2, 5))):
        kind = pick("parallel", "parallel_2", "gla")
        if kind == "gla":
            mx = {"heads": pick(1, 2, 3), "dim": pick(8, 20, 32), "vdim": pick(8, 24, 32), "tau": pick(1.0, 4.0, 16.0)}
        elif kind == "parallel":
            mx = par(attention(), pick(24, 40, 64), pick(3, 8, 16, 33), pick(1, 4, 8), pick(1, 2, 4), float(rng.uniform(0.3, 1.5)),
                     float(rng.uniform(0.3, 1.5)))
        else:
            groups = pick(1, 2)
            heads = groups * pick(1, 2, 3)
            vdim = pick(8, 16, 24)
            mx = par2(attention(), heads, vdim, pick(4, 16, 24), groups, pick(1, heads, 2 if (heads * vdim) % 2 == 0 else 1),
                      pick(2, 3, 4))
        layers.append(layer(kind, mx, mlp()))
    return {"architecture": "Meropel", "vocab": int(rng.integers(50, 300)), "width": pick(64, 72, 100, 128),
            "norm": {"eps": pick(1e-5, 1e-6)}, "logit_scale": pick(1.0, 0.3, 2.0),
            "embedding": {"bigram": {"buckets": int(rng.integers(3, 200)), "mul_prev": int(rng.integers(1, 1000)),
                                     "mul_cur": int(rng.integers(1, 1000))}},
            "layers": layers}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [301, 302, 304, 305, 306, 307, 308, 309])
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    raw = random_config(seed)
    folder = write_model(str(tmp_path / "m"), raw, seed)
    reqs = requests_for(raw, [90, 37, 3], seed=seed)
    engine = engine_for(folder, dtype)
    for recs in (traces.whole(reqs), traces.batches(reqs, 3, first_part=lambda n: max(1, n - 20))):
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
        g.attach_storage(torch.full(g.storage_shape(), float("nan"), dtype=dtype, device=DEV),   # an unwritten row that is read shows
                         torch.full(g.value_storage_shape(), float("nan"), dtype=dtype, device=DEV))
    cache.state = torch.full((cache.max_slots, max(cache.state_bytes_per_slot, 1)), 0x7f, dtype=torch.uint8, device=DEV)
    cache.zero_state = lambda slot: cache.state[slot].zero_()     # as the engine does when a slot is handed out
    return cache


def summed(o):
    """A mixer's update as one tensor: partial sums added, the terms of a combined update formed as their kernel forms them."""
    if torch.is_tensor(o):
        return (o.sum(0) if o.dim() == 3 else o).float()
    total = 0
    for t in o:
        v = summed(t.value).double()
        if t.norm_weight is not None:
            v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + t.norm_eps) * t.norm_weight.double()
        if t.row_scale is not None:
            v = v * t.row_scale.double()[:, None]
        total = total + t.scale * v
    return total.float()


def run_in_steps(mixer, rt, cache, h, cuts):
    """The mixer's output for one sequence whose rows h come in steps that end at the given cuts."""
    from odin_infer_b200.engine.step import StepBatch, StepEntry
    slot = cache.take_slot()
    outs, at = [], 0
    for end in cuts:
        st = cache.extend(slot, end - at)
        step = StepBatch(cache, [StepEntry(slot, [0] * (end - at), list(range(end - at)))], [st], DEV)
        outs.append(summed(mixer.forward(rt, step, h[at:end].contiguous(), 0)).clone())
        cache.after_step(slot)
        at = end
    cache.give_back_slot(slot)
    return torch.cat(outs)


def bound(part, dtype, rt, seed, prefix="m."):
    """The part bound to weights of the tests' making; returns the weights in float64 by name."""
    gen = torch.Generator().manual_seed(seed)
    t = {p.name: make_weight(p.name, p.concrete_shape, gen).to(torch.bfloat16).to(dtype).to(DEV) for p in part.params()}
    ref = {k: v.double().cpu() for k, v in t.items()}
    part.bind(dict(t), rt)
    return ref


CUTS = lambda n: ([n], [2, 4, 7, 8, 64, 65, n - 3, n], list(range(n - 40, n + 1)), [1, 2, 3, n])  # noqa: E731


SCAN_GEOMETRIES = [  # inner, state, dt_rank, taps, tokens
    (48, 8, 4, 4, 150), (40, 33, 1, 2, 131), (72, 16, 6, 1, 90), (36, 70, 3, 5, 300), (256, 16, 8, 4, 520), (24, 200, 2, 3, 270)]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("geom", SCAN_GEOMETRIES)
def test_selective_scan_alone_remembers_a_loud_token(dtype, tol, geom):
    """Token 5 is thirty times louder than the rest: channels whose step sizes are small still carry it a hundred tokens
    later, and a state or a convolution's memory that is lost between steps changes the rows after the cut.  Whole, in
    portions down to one token (shorter than the convolution), and the last forty tokens one by one."""
    from odin_infer_b200.parts import PartSpec, build_part
    inner, N, R, taps, n = geom
    width = 80
    rt = runtime(dtype)
    names = {"in": "m.in", "conv": "m.conv", "conv_bias": "m.conv.b", "x": "m.x", "dt": "m.dt", "dt_bias": "m.dt.b",
             "A_log": "m.A_log", "D": "m.D", "o": "m.o"}
    scan = build_part("mixer", PartSpec("selective_scan", dict(width=width, inner=inner, state=N, dt_rank=R, taps=taps, names=names)))
    w = bound(scan, dtype, rt, inner + N)
    torch.manual_seed(N)
    h = torch.randn(n, width, device=DEV)
    h[5] *= 30.0
    h = h.to(dtype)
    mx = {"inner": inner, "state": N, "dt_rank": R, "conv": taps}
    ref = P.selective_scan(h.double().cpu(), w, "m.", mx)
    quiet = h.clone()
    quiet[5] /= 30.0
    other = P.selective_scan(quiet.double().cpu(), w, "m.", mx)
    assert (other[80] - ref[80]).abs().max() > 1e-3 * ref[80].abs().max()     # the loud token is still heard at row 80
    cache = cache_for([scan], dtype)
    for cuts in CUTS(n):
        close(run_in_steps(scan, rt, cache, h, cuts), ref, tol)
    close(run_in_steps(scan, rt, cache, quiet, [n]), other, tol)   # the slot's state was cleared for the next sequence


DUAL_GEOMETRIES = [  # heads, head size, state, groups, norm groups, taps, tokens
    (4, 16, 24, 2, 4, 4, 150), (1, 36, 9, 1, 1, 1, 131), (6, 8, 64, 3, 2, 2, 90), (8, 32, 64, 2, 2, 4, 520), (3, 40, 130, 1, 3, 3, 70)]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("geom", DUAL_GEOMETRIES)
def test_state_space_dual_alone(dtype, tol, geom):
    """As above for the recurrence over heads: heads of one group share B and C, every head has its own decay and step."""
    from odin_infer_b200.parts import PartSpec, build_part
    H, Pd, N, G, NG, taps, n = geom
    width = 80
    rt = runtime(dtype)
    names = {"in": "m.in", "conv": "m.conv", "conv_bias": "m.conv.b", "dt_bias": "m.dt_bias", "A_log": "m.A_log", "D": "m.D",
             "norm": "m.norm", "o": "m.o"}
    ssd = build_part("mixer", PartSpec("state_space_dual", dict(width=width, n_heads=H, head_dim=Pd, state=N, groups=G,
                                                                norm_groups=NG, taps=taps, eps=1e-5, names=names)))
    w = bound(ssd, dtype, rt, H * 10 + N)
    torch.manual_seed(N)
    h = torch.randn(n, width, device=DEV)
    h[5] *= 10.0
    h = h.to(dtype)
    mx = {"heads": H, "vdim": Pd, "state": N, "groups": G, "norm_groups": NG, "conv": taps}
    ref = P.state_space_dual(h.double().cpu(), w, "m.", mx, 1e-5)
    cache = cache_for([ssd], dtype)
    for cuts in CUTS(n):
        close(run_in_steps(ssd, rt, cache, h, cuts), ref, tol)
    quiet = h.clone()
    quiet[5] /= 10.0
    close(run_in_steps(ssd, rt, cache, quiet, [n]), P.state_space_dual(quiet.double().cpu(), w, "m.", mx, 1e-5), tol)


GLA_GEOMETRIES = [(3, 20, 28, 8.0, 150), (1, 36, 12, 1.0, 131), (2, 64, 128, 16.0, 520), (4, 130, 16, 64.0, 90)]  # heads, dim, vdim, tau, tokens


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("geom", GLA_GEOMETRIES)
def test_gated_linear_attention_alone(dtype, tol, geom):
    """With a large tau the state forgets slowly: a loud token at the start is still heard at the end; with tau = 1 it is
    forgotten within a few tokens.  Whole, in portions, one by one."""
    from odin_infer_b200.parts import PartSpec, build_part
    H, D, V, tau, n = geom
    width = 80
    rt = runtime(dtype)
    names = {k: "m." + k for k in ("q", "k", "v", "g", "o", "norm", "a1", "a2")}
    names["a2_bias"] = "m.a2.b"
    gla = build_part("mixer", PartSpec("gated_linear_attention", dict(width=width, n_heads=H, head_dim=D, v_head_dim=V, tau=tau,
                                                                      eps=1e-5, decay_rank=6, names=names)))
    w = bound(gla, dtype, rt, H * 7 + D)
    torch.manual_seed(D)
    h = torch.randn(n, width, device=DEV)
    h[3] *= 20.0
    h = h.to(dtype)
    mx = {"heads": H, "dim": D, "vdim": V, "tau": tau}
    ref = P.gated_linear_attention(h.double().cpu(), w, "m.", mx, 1e-5)
    cache = cache_for([gla], dtype)
    for cuts in CUTS(n):
        close(run_in_steps(gla, rt, cache, h, cuts), ref, tol)


ATTENTION_GEOMETRIES = [  # variant, heads, kv heads, dim, vdim, rot, tokens
    ("parallel", 4, 2, 24, 40, 8, 200), ("parallel", 2, 2, 16, 8, 0, 131), ("parallel", 4, 2, 64, 64, 32, 330),
    ("parallel_2", 4, 1, 32, 32, 32, 200), ("parallel_2", 3, 3, 20, 28, 12, 131), ("parallel_2", 2, 1, 128, 128, 64, 330),
    ("parallel_2", 8, 2, 64, 64, 64, 130)]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("geom", ATTENTION_GEOMETRIES)
def test_attention_branches_alone_with_a_loud_key_far_back(dtype, tol, geom):
    """Both attention branches (the gate per head; biases, the norm over the whole projections and the rotation in pairs)
    against the plain attention, whole, in portions and one by one, over page borders.  Token 2's row is made loud, so that
    its key draws weight from hundreds of tokens away in the first variant (the second norms it away: there the loud row
    checks the norm over the whole projection)."""
    from odin_infer_b200.parts import PartSpec, build_part
    variant, H, G, D, V, rot, n = geom
    width, base, scale = 80, 700.0, 0.21
    rt = runtime(dtype)
    names = {k: "m." + k for k in ("q", "k", "v", "o")}
    more = dict(qk_norm=False, gate="m.g", gate_per_head=True)
    if variant == "parallel_2":
        names.update({"q_norm": "m.q.norm", "k_norm": "m.k.norm"})
        more = dict(qk_norm="whole", biases={"q": "m.q.b", "k": "m.k.b", "v": "m.v.b"})
    layout = "pairs" if variant == "parallel_2" else "halves"
    att = build_part("mixer", PartSpec("gqa_attention", dict(width=width, n_q_heads=H, n_kv_heads=G, head_dim=D, v_head_dim=V,
                                                             position_encoding="pe" if rot else None, eps=1e-5, scale=scale,
                                                             names=names, **more)))
    if rot:
        att.pe = build_part("position_encoding", PartSpec("rope", dict(rotary_dim=rot, theta=base, precise=True, layout=layout,
                                                                       exact_angles=True)))
        att.pe.prepare(rt, n)
    w = bound(att, dtype, rt, H * 13 + D)
    torch.manual_seed(D + V)
    h = torch.randn(n, width, device=DEV)
    h[2] *= 6.0
    h = h.to(dtype)
    mx = attn(H, G, D, V, scale, rot=rot, base=base)
    ref = P.attention_left(h.double().cpu(), w, "m.", mx, 1e-5, list(range(n)), variant)
    cache = cache_for([att], dtype)
    for cuts in ([n], [2, 63, 64, 65, n - 3, n], list(range(n - 40, n + 1))):
        close(run_in_steps(att, rt, cache, h, cuts), ref, tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("norms", [False, True])
def test_two_mixers_side_by_side(dtype, tol, norms):
    """The two ways of putting the branches together: a sum with two factors, and half the sum of the two outputs after
    each has passed an RMSNorm over the width."""
    from odin_infer_b200.parts import PartSpec, build_part
    width, n = 80, 140
    rt = runtime(dtype)
    left = PartSpec("gqa_attention", dict(width=width, n_q_heads=2, n_kv_heads=1, head_dim=16, v_head_dim=24, eps=1e-5, scale=0.25,
                                          qk_norm=False, names={k: "m.left." + k for k in "qkvo"}))
    right = PartSpec("gated_linear_attention", dict(width=width, n_heads=2, head_dim=12, v_head_dim=20, tau=4.0, eps=1e-5,
                                                    decay_rank=5, names={**{k: "m.right." + k for k in ("q", "k", "v", "g", "o", "norm", "a1", "a2")},
                                                                         "a2_bias": "m.right.a2.b"}))
    both = build_part("mixer", PartSpec("side_by_side", dict(left=left, right=right, width=width, left_scale=0.5 if norms else 0.7,
                                                            right_scale=0.5 if norms else 1.9, eps=1e-5,
                                                            norms={"left": "m.left.out", "right": "m.right.out"} if norms else None)))
    w = bound(both, dtype, rt, 77)
    torch.manual_seed(5)
    h = torch.randn(n, width, device=DEV).to(dtype)
    hd = h.double().cpu()
    a = P.causal_softmax_attention((hd @ w["m.left.q"].T).view(n, 2, 16), (hd @ w["m.left.k"].T).view(n, 1, 16),
                                   (hd @ w["m.left.v"].T).view(n, 1, 24), 0.25).reshape(n, 48) @ w["m.left.o"].T
    b = P.gated_linear_attention(hd, w, "m.right.", {"heads": 2, "dim": 12, "vdim": 20, "tau": 4.0}, 1e-5)
    ref = 0.5 * (P.rms(a, w["m.left.out"], 1e-5) + P.rms(b, w["m.right.out"], 1e-5)) if norms else 0.7 * a + 1.9 * b
    cache = cache_for([both], dtype)
    for cuts in ([n], [2, 64, 65, n], list(range(n - 30, n + 1))):
        close(run_in_steps(both, rt, cache, h, cuts), ref, tol)


def test_pair_table_embedding_carries_the_token_before():
    """The hashed row of (token before, token): inside a step from the row above, across steps from the state, for a
    sequence's first token the table's last row; two sequences in one step, a slot used again."""
    from odin_infer_b200.cache import CacheManager
    from odin_infer_b200.engine.step import StepBatch, StepEntry
    from odin_infer_b200.parts import PartSpec, build_part
    V, d, buckets, mp, mc = 50, 24, 13, 1000003, 77
    rt = runtime(torch.float32)
    emb = build_part("embedding", PartSpec("token_table", dict(vocab_size=V, width=d, weight="embed",
                                                               pair={"weight": "pairs", "buckets": buckets, "mul_prev": mp, "mul_cur": mc})))
    torch.manual_seed(0)
    t = {"embed": torch.randn(V, d, device=DEV), "pairs": torch.randn(buckets + 1, d, device=DEV)}
    emb.bind(dict(t), rt)
    cache = CacheManager(64 * 8, 64 * 4)
    emb.state_entry = cache.add_entry(None, emb.state_bytes())
    cache.entry_writes = [False]
    cache.state = torch.full((cache.max_slots, cache.state_bytes_per_slot), 0x7f, dtype=torch.uint8, device=DEV)
    cache.zero_state = lambda slot: cache.state[slot].zero_()
    seqs = {0: random_tokens(9, V, 1), 1: random_tokens(5, V, 2)}
    ref = {k: P.embed(v, t["embed"].double().cpu(), t["pairs"].double().cpu(), {"buckets": buckets, "mul_prev": mp, "mul_cur": mc})
           for k, v in seqs.items()}
    for _ in range(2):   # the second round uses the slots again
        slots = {k: cache.take_slot() for k in seqs}
        at = {k: 0 for k in seqs}
        for sizes in ({0: 4, 1: 1}, {0: 1, 1: 1}, {0: 4, 1: 3}):
            entries, starts = [], []
            for k, m in sizes.items():
                starts.append(cache.extend(slots[k], m))
                entries.append(StepEntry(slots[k], seqs[k][at[k]:at[k] + m], []))
            x = emb.forward(rt, StepBatch(cache, entries, starts, DEV))
            r = 0
            for k, m in sizes.items():
                close(x[r:r + m], ref[k][at[k]:at[k] + m], 1e-6)
                r, at[k] = r + m, at[k] + m
        for s in slots.values():
            cache.give_back_slot(s)


@pytest.mark.parametrize("E,ident,groups,keep,top", [(6, 3, 3, 2, 3), (8, 2, 2, 1, 4), (4, 0, 1, 1, 1), (3, 1, 4, 4, 4), (16, 0, 4, 2, 4),
                                                      (20, 12, 32, 5, 5), (5, 1, 2, 2, 2)])
@pytest.mark.parametrize("given_logits", [False, True])
def test_router_with_corrected_scores_in_groups(E, ident, groups, keep, top, given_logits):
    """Choice by score + correction inside the groups that stay (a group's score its largest choice score, also when all
    are negative), weights from the scores without it; rows without an expert come back as one summed weight."""
    from odin_infer_b200.csrc import ops
    T, d, rows = 64, 48, E + ident
    torch.manual_seed(E * 100 + groups)
    h = torch.randn(T, d, device=DEV)
    wr = 3.0 * torch.randn(rows, d, device=DEV) / math.sqrt(d)
    corr = 0.3 * torch.randn(rows, device=DEV) - 0.5      # mostly negative choice scores: a masked group must not win with 0
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
    passed = torch.empty(T, dtype=torch.float32, device=DEV)
    logits = (h @ wr.T).contiguous() if given_logits else None
    ops.moe_router(h, wr, corr, top, 0, None, ids, wts, logits, score="softmax_corrected_in_groups", groups=groups, keep=keep,
                   route_scale=1.7, n_real=E, pass_out=passed)
    picks = P.route(h.double().cpu(), wr.double().cpu(), corr.double().cpu(),
                    {"experts": E, "identity": ident, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}})
    for t in range(T):
        want_real = sorted((e, w) for e, w in picks[t] if e < E)
        got_real = sorted((int(e), float(w)) for e, w in zip(ids[t].tolist(), wts[t].tolist()) if e >= 0)
        assert [e for e, _ in want_real] == [e for e, _ in got_real], (t, picks[t], ids[t].tolist())
        for (_, a), (_, b) in zip(want_real, got_real):
            assert abs(a - b) <= 1e-5 * 1.7
        assert abs(sum(w for e, w in picks[t] if e >= E) - float(passed[t])) <= 1e-5 * 1.7
        assert sum(1 for e in ids[t].tolist() if e < 0) == sum(1 for e, _ in picks[t] if e >= E)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2.5e-2)])
@pytest.mark.parametrize("T", [7, 200])
@pytest.mark.parametrize("E,ident,groups,keep,top,ff,shared", [(6, 3, 3, 2, 3, 40, 80), (8, 2, 2, 1, 4, 32, 56), (4, 0, 1, 1, 4, 24, 0),
                                                              (3, 2, 5, 2, 1, 16, 16)])
def test_feed_forward_of_experts_with_rows_that_hand_the_input_through(dtype, tol, T, E, ident, groups, keep, top, ff, shared):
    from odin_infer_b200.engine.step import StepBatch, StepEntry
    from odin_infer_b200.cache import CacheManager
    from odin_infer_b200.parts import PartSpec, build_part
    width = 64
    rt = runtime(dtype)
    f = "m."
    names = {"router": f + "router", "router_bias": f + "correction", "gate": f + "e{e}.gate", "up": f + "e{e}.up", "down": f + "e{e}.down",
             "shared_gate": f + "shared.gate", "shared_up": f + "shared.up", "shared_down": f + "shared.down"}
    part = build_part("feed_forward", PartSpec("routed_experts", dict(
        width=width, inner=ff, n_experts=E, top=top, shared_inner=shared, score="softmax_corrected_in_groups", groups=groups,
        keep=keep, route_scale=1.3, n_pass=ident, names=names)))
    w = bound(part, dtype, rt, E * 31 + T)
    torch.manual_seed(T)
    h = torch.randn(T, width, device=DEV).to(dtype)
    mlp = moe(E, ident, top, ff, groups, keep, 1.3, shared=shared)
    ref = P.expert_mlp(h.double().cpu(), w, "m.", mlp)
    cache = CacheManager(64 * 8, 64 * 8)
    slot = cache.take_slot()
    cache.extend(slot, T)
    step = StepBatch(cache, [StepEntry(slot, [0] * T, [])], [0], DEV)
    got = summed(part.forward(rt, step, h))
    if dtype == torch.float32:
        close(got, ref, tol)
    else:   # a close call of the router may fall the other way for a token or two
        err = (got.double().cpu() - ref).abs().max(dim=1).values / ref.abs().max()
        assert int((err > tol).sum()) <= max(1, T // 20), err.max()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("d,rows", [(96, 9), (100, 3), (2048, 5)])
def test_terms_are_summed_normed_added_and_normed_again(dtype, tol, d, rows):
    """The kernel behind a block's second norms: partial sums, a term with a norm of its own and a factor, a term with a
    number per row; then the update's norm, the add into the residual stream, and the next norm's output; also with
    gathered rows (the stream is then left alone) and as a plain sum."""
    from odin_infer_b200.csrc import ops
    torch.manual_seed(d)
    x = torch.randn(rows, d, device=DEV)
    a = torch.randn(3, rows, d, device=DEV)
    b = torch.randn(rows, d, device=DEV).to(dtype)
    c = torch.randn(rows, d, device=DEV).to(dtype)
    per_row = torch.rand(rows, device=DEV)
    wn, wp, wx = (1.0 + 0.3 * torch.randn(d, device=DEV)).to(dtype), (1.0 + 0.3 * torch.randn(d, device=DEV)).to(dtype), \
        (1.0 + 0.3 * torch.randn(d, device=DEV)).to(dtype)
    terms = [ops.Term(a, 0.7), ops.Term(b, 0.5, None, wn, 1e-5), ops.Term(c, 1.0, per_row)]
    y = 0.7 * a.double().sum(0) + 0.5 * P.rms(b.double(), wn.double(), 1e-5) + c.double() * per_row.double()[:, None]
    x_new = x.double() + P.rms(y, wp.double(), 1e-6)
    want = P.rms(x_new, wx.double(), 1e-5)
    x1, out = x.clone(), torch.empty(rows, d, dtype=dtype, device=DEV)
    ops.combine_add(x1, terms, wp, 1e-6, wx, 1e-5, out)
    close(x1, x_new, 2e-6)
    close(out, want, tol)
    pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    x2, out2 = x.clone(), torch.empty(2, d, dtype=dtype, device=DEV)
    ops.combine_add(x2, terms, wp, 1e-6, wx, 1e-5, out2, rows=pick)
    assert torch.equal(x2, x) and torch.equal(out2, out[pick.long()])
    plain = torch.empty(rows, d, dtype=torch.float32, device=DEV)
    ops.combine_add(None, terms, out=plain)
    close(plain, y, 2e-6)
    x3 = x.clone()
    ops.combine_add(x3, terms)
    close(x3, x.double() + y, 2e-6)
