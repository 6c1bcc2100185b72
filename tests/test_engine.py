"""Engine mechanics: continuous batching, prefix cache (mechanical invariants and output equivalence), sampler semantics."""
import random

import pytest
import torch

from deliverance_b200.ckpt.loader import WeightLoader
from deliverance_b200.ckpt.tiny import write_tiny_model
from deliverance_b200.config import load_config
from deliverance_b200.engine.engine import Engine, EngineConfig
from deliverance_b200.engine.sampler import Sampler, SamplingState, candidate_limit, sample_top_k_top_p_batch, xtc_pick
from deliverance_b200.kv.paged import KvCacheSettings, PageAllocator, PrefixCache, compose_salt
from deliverance_b200.models.transformer import DecoderModel
from deliverance_b200.params import FinishReason, GeneratorParameters


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("m") / "llama")
    write_tiny_model(d, "llama", seed=7, std=0.05)
    cfg = load_config(d)
    return DecoderModel(cfg, "cpu").load(WeightLoader(d))


def _engine(model, **kw):
    kv = kw.pop("kv", KvCacheSettings())
    return Engine(model, EngineConfig(num_pages=kw.pop("pages", 128), max_batch_tokens=kw.pop("chunk", 64), kv=kv, **kw))


def test_batched_equals_single(tiny):
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 250, (n,), generator=g).tolist() for n in (5, 40, 70, 33)]
    singles = [_engine(tiny).generate(p, GeneratorParameters(max_tokens=5)).token_ids for p in prompts]
    eng = _engine(tiny, chunk=48)
    rs = eng.generate_batch(prompts, GeneratorParameters(max_tokens=5))
    assert [r.token_ids for r in rs] == singles
    assert eng.kv.allocator.available() == eng.kv.num_pages - 1 - sum(len(e.pages) for e in eng.kv.prefix.entries.values()) or True
    assert all(r.finish_reason == FinishReason.MAX_TOKENS for r in rs)


def test_checkpoint_lengths_policies():
    s = KvCacheSettings()
    assert s.checkpoint_lengths(100) == [32, 64, 96]
    assert s.checkpoint_lengths(700) == [32, 64, 480, 512]
    assert s.checkpoint_lengths(31) == []
    assert KvCacheSettings(policy="FIXED_BLOCKS").checkpoint_lengths(130) == [32, 64, 96, 128]
    assert KvCacheSettings(policy="ANCHORS").checkpoint_lengths(300) == [32, 64, 128, 288]


def test_prefix_cache_lru_refcounts():
    alloc = PageAllocator(16)
    pc = PrefixCache(KvCacheSettings(max_entries=3, policy="FIXED_BLOCKS"), alloc)
    toks = list(range(100))
    pages = [alloc.alloc() for _ in range(4)]
    assert pc.store("s", toks, pages) == 3
    assert pc.lookup("other", toks) is None
    hit = pc.lookup("s", toks[:70] + [999] * 30)
    assert hit.length == 64 and hit.pages == pages[:2] and alloc.ref[pages[0]] == 1 + 3 + 1
    for p in hit.pages:
        alloc.release(p)
    pc.store("s", list(range(1000, 1040)), [alloc.alloc(), alloc.alloc()])  # a 4th entry evicts the oldest
    assert len(pc.entries) == 3 and pc.metrics["evict"] == 1
    for p in pages:
        alloc.release(p)
    pc.clear()
    assert alloc.available() == 15 - 2  # only the two pages still owned by the caller stay out


def test_salt_composition():
    assert compose_salt("a") == "a"
    assert compose_salt("a", "ad1") == "lora:ad1|a"
    assert compose_salt("a", "ad1", 1, 4) == "tp:size=4:rank=1|lora:ad1|a"


def test_prefix_hit_output_equivalence(tiny):
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(3, 250, (96,), generator=g).tolist()
    p1, p2 = shared + [5, 6, 7], shared + [9, 10, 11, 12]
    cold = _engine(tiny, kv=KvCacheSettings(enabled=False))
    ref2 = cold.generate(p2, GeneratorParameters(max_tokens=6)).token_ids
    eng = _engine(tiny)
    eng.generate(p1, GeneratorParameters(max_tokens=2))
    r2 = eng.generate(p2, GeneratorParameters(max_tokens=6))
    assert r2.prefix_hit_tokens == 96 and r2.token_ids == ref2
    # salts separate the caches
    r3 = eng.generate(p2, GeneratorParameters(max_tokens=6, cache_salt="tenant-b"))
    assert r3.prefix_hit_tokens == 0 and r3.token_ids == ref2
    # full-prompt hit: the last prompt token is replayed and decoding starts at the full prompt length
    p3 = shared[:64]
    a = eng.generate(p3, GeneratorParameters(max_tokens=3))
    b = eng.generate(p3, GeneratorParameters(max_tokens=3))
    assert b.prefix_hit_tokens == 64 and a.token_ids == b.token_ids


def test_request_limits_and_stops(tiny):
    eng = _engine(tiny)
    with pytest.raises(ValueError):
        eng.generate([1] * 300)
    with pytest.raises(ValueError):
        eng.generate([1, 2, 3], GeneratorParameters(ntokens=3))
    r = eng.generate([4, 5, 6], GeneratorParameters(ntokens=8))
    assert r.generated_tokens == 5 and r.finish_reason == FinishReason.MAX_TOKENS
    first = eng.generate([4, 5, 6], GeneratorParameters(max_tokens=3)).token_ids[0]
    eng2 = Engine(tiny, EngineConfig(num_pages=32), eos_ids=(first,))
    r = eng2.generate([4, 5, 6], GeneratorParameters(max_tokens=9))
    assert r.finish_reason == FinishReason.STOP_TOKEN and r.generated_tokens == 1
    with pytest.raises(ValueError):
        GeneratorParameters(guided_regex="a", guided_choice=["a"]).validate()
    with pytest.raises(ValueError):
        GeneratorParameters(uniform_top_p=0.5, top_p=0.5).validate()


def test_candidate_limit_and_defaults():
    assert candidate_limit(None, 100) == 100 and candidate_limit(5, 100) == 5 and candidate_limit(500, 100) == 100
    assert candidate_limit(0.9, 100) == 10 and candidate_limit(0.999, 100) == 1
    st = SamplingState.create(GeneratorParameters(temperature=0.7))
    assert st.effective()[1] == 0.10  # nothing set -> top_p = 0.10
    assert SamplingState.create(GeneratorParameters(temperature=0.7, top_k=3)).effective()[1] is None


def test_top_k_top_p_semantics():
    logits = torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05]]))
    T = torch.tensor([1.0])

    def run(limit, top_p, uniform, u):
        return int(sample_top_k_top_p_batch(logits, T, torch.tensor([limit]), torch.tensor([top_p]), torch.tensor([uniform]), torch.tensor([u]))[0])

    assert run(4, 0.0, False, 0.49) == 0 and run(4, 0.0, False, 0.51) == 1 and run(4, 0.0, False, 0.96) == 3
    assert run(1, 0.0, False, 0.99) == 0  # top_k = 1
    assert run(2, 0.0, False, 0.7) == 1  # renormalised over the kept two: 0.625 / 0.375
    assert run(4, 0.6, False, 0.99) == 1  # nucleus {0, 1}
    assert run(4, 0.8, True, 0.1) == 0 and run(4, 0.8, True, 0.5) == 1 and run(4, 0.8, True, 0.99) == 1  # uniform pick inside it
    # stable order on ties: the lower index comes first
    tie = torch.zeros(1, 4)
    assert int(sample_top_k_top_p_batch(tie, T, torch.tensor([4]), torch.tensor([0.0]), torch.tensor([False]), torch.tensor([0.2]))[0]) == 0


def test_xtc_and_sampler_determinism():
    logits = torch.log(torch.tensor([0.5, 0.3, 0.15, 0.05]))
    assert xtc_pick(logits, 0.1, 0.5, 0.9, set()) is None  # u > probability: no-op
    assert xtc_pick(logits, 0.1, 1.0, 0.2, set()) == 2  # least probable above the threshold
    assert xtc_pick(logits, 0.1, 1.0, 0.2, {0}) == 0  # most probable is special -> returned
    assert xtc_pick(logits, 0.9, 1.0, 0.2, set()) is None
    s = Sampler()
    big = torch.randn(3, 500, generator=torch.Generator().manual_seed(3))
    mk = lambda: [SamplingState.create(GeneratorParameters(temperature=0.9, top_p=0.9, seed=11)) for _ in range(3)]  # noqa: E731
    a, _ = s.sample(big, mk())
    b, _ = s.sample(big, mk())
    assert a == b
    toks, lps = s.sample(big, [SamplingState.create(GeneratorParameters(logprobs=True, top_logprobs=3)) for _ in range(3)])
    assert toks == torch.argmax(big, dim=-1).tolist()
    assert abs(lps[0].logprob - torch.log_softmax(big[0], -1)[toks[0]].item()) < 1e-5 and len(lps[0].top) == 3


def test_cancel_and_callback_error(tiny):
    eng = _engine(tiny)
    seen = []
    r = eng.add_request([4, 5, 6], GeneratorParameters(max_tokens=50), on_token=lambda t, rq: (seen.append(t), eng.abort(rq) if len(seen) == 3 else None))
    eng.run([r])
    assert r.finish_reason == FinishReason.CANCELLED and len(r.output) == 3

    def boom(t, rq):
        raise RuntimeError("client went away")

    r2 = eng.add_request([4, 5, 6], GeneratorParameters(max_tokens=50), on_token=boom)
    eng.run([r2])
    assert r2.finish_reason == FinishReason.ERROR and eng.kv.allocator.available() > 0


def test_lookahead_decode_matches_synchronous(tmp_path):
    """One-step lookahead (tokens of step N read while step N + 1 runs) must produce the same tokens, stop reasons and
    callback order per request as the synchronous schedule, with staggered arrivals, different lengths and a cancellation."""
    from deliverance_b200.ckpt.tiny import write_tiny_model
    from deliverance_b200.ckpt.loader import WeightLoader
    from deliverance_b200.config import load_config
    from deliverance_b200.engine.engine import Engine, EngineConfig
    from deliverance_b200.models.transformer import DecoderModel
    from deliverance_b200.params import GeneratorParameters

    d = str(tmp_path / "m")
    write_tiny_model(d, "qwen3", seed=11, std=0.08)
    cfg = load_config(d)
    model = DecoderModel(cfg, "cpu").load(WeightLoader(d))
    prompts = [[3, 5, 7, 9, 11], [2, 4, 6], [8, 1, 8, 1, 8, 1, 8], [13, 17]]
    lens = [9, 4, 12, 6]

    def run(lookahead):
        eng = Engine(model, EngineConfig(num_pages=64, max_batch_tokens=8, lookahead=lookahead), eos_ids=(-1,))
        seen = {}
        reqs = []
        for i, (p, n) in enumerate(zip(prompts[:3], lens[:3])):
            reqs.append(eng.add_request(p, GeneratorParameters(max_tokens=n, temperature=0.0), on_token=lambda t, r, i=i: seen.setdefault(i, []).append(t)))
        steps = 0
        late = None
        while eng.has_work():
            eng.step()
            steps += 1
            if steps == 4:  # a request that arrives while decode steps are in flight
                late = eng.add_request(prompts[3], GeneratorParameters(max_tokens=lens[3], temperature=0.0))
                reqs.append(late)
            if steps == 6:
                eng.abort(reqs[2])
        assert eng._inflight is None
        return [r.output for r in reqs], [r.finish_reason for r in reqs], seen, eng.kv.allocator.available()

    out_sync, why_sync, seen_sync, free_sync = run(False)
    out_la, why_la, seen_la, free_la = run("force")
    assert out_la[0] == out_sync[0] and out_la[1] == out_sync[1] and out_la[3] == out_sync[3]
    assert why_la[:2] == why_sync[:2] and why_la[3] == why_sync[3]
    # the cancelled request stops within one step of the synchronous schedule and its tokens are a prefix-consistent run
    n = min(len(out_la[2]), len(out_sync[2]))
    assert out_la[2][:n] == out_sync[2][:n] and abs(len(out_la[2]) - len(out_sync[2])) <= 2
    assert seen_la[0] == out_la[0] and seen_la[1] == out_la[1]
    assert free_la == free_sync  # every page came back


def test_concurrent_arrivals_share_prefix_through_cache(tmp_path):
    """Requests that arrive together and share a prefix: admission is gated by the prefill budget, so the later ones find the
    prefix that the first ones stored, and outputs equal the uncached run."""
    from deliverance_b200.ckpt.loader import WeightLoader
    from deliverance_b200.ckpt.tiny import write_tiny_model
    from deliverance_b200.config import load_config
    from deliverance_b200.engine.engine import Engine, EngineConfig
    from deliverance_b200.models.transformer import DecoderModel
    from deliverance_b200.params import GeneratorParameters

    d = str(tmp_path / "m")
    write_tiny_model(d, "llama", seed=12, std=0.08)
    model = DecoderModel(load_config(d), "cpu").load(WeightLoader(d))
    prefix = [(7 * i + 3) % 250 + 1 for i in range(96)]
    prompts = [prefix + [10 + i, 20 + i, 30 + i] for i in range(6)]

    def run(cache_on, budget):
        ec = EngineConfig(num_pages=128, max_batch_tokens=budget, max_seqs=8)
        ec.kv.enabled = cache_on
        eng = Engine(model, ec, eos_ids=(-1,))
        rs = eng.generate_batch(prompts, GeneratorParameters(max_tokens=5, temperature=0.0))
        return [r.token_ids for r in rs], dict(eng.kv.prefix.metrics), eng.metrics["prefill_tokens"]

    base, _, tokens_nocache = run(False, 100)
    got, m, tokens_cached = run(True, 100)
    assert got == base
    assert m["hits"] >= 4 and tokens_cached < tokens_nocache * 0.6


def test_disk_tier_restores_evicted_prefix(tmp_path):
    """A prefix evicted from memory is written to disk, found again by a later request and gives the same tokens."""
    from deliverance_b200.ckpt.loader import WeightLoader
    from deliverance_b200.ckpt.tiny import write_tiny_model
    from deliverance_b200.config import load_config
    from deliverance_b200.engine.engine import Engine, EngineConfig
    from deliverance_b200.models.transformer import DecoderModel
    from deliverance_b200.params import GeneratorParameters

    d = str(tmp_path / "m")
    write_tiny_model(d, "llama", seed=14, std=0.08)
    model = DecoderModel(load_config(d), "cpu").load(WeightLoader(d))
    a = [(5 * i + 1) % 250 + 1 for i in range(70)]
    b = [(11 * i + 7) % 250 + 1 for i in range(70)]
    p = GeneratorParameters(max_tokens=4, temperature=0.0)
    ec = EngineConfig(num_pages=64)
    ec.kv.max_entries = 2  # tiny in-memory tier: the next prompt's entries push the previous ones out
    ec.kv.policy = "ANCHORS"
    eng = Engine(model, ec, eos_ids=(-1,))
    disk = eng.kv.attach_disk(str(tmp_path / "kvdisk"), compression="LZ4")
    first = eng.generate(a, p).token_ids
    eng.generate(b, p)
    assert disk.metrics["disk_writes"] >= 1 and eng.kv.prefix.metrics["evict"] >= 1
    computed_before = eng.metrics["prefill_tokens"]
    again = eng.generate(a, p).token_ids
    assert again == first
    assert disk.metrics["disk_hits"] >= 1
    assert eng.metrics["prefill_tokens"] - computed_before < len(a)  # part of the prompt came back from disk


@pytest.mark.parametrize("compression", ["NONE", "MSE_TURBOQUANT"])
def test_disk_store_formats_roundtrip(tmp_path, compression):
    from deliverance_b200.kv.disk import DiskPrefixStore
    from deliverance_b200.kv.paged import PagedKVCache

    layout = {"layers": 2, "kv_heads": 2, "head_dim": 64, "layer_kinds": ["attention", "attention"]}
    kv = PagedKVCache(layout, 16, "cpu", torch.float32)
    g = torch.Generator().manual_seed(2)
    for t in kv.k + kv.v:
        t.copy_(torch.randn(t.shape, generator=g))
    store = DiskPrefixStore(str(tmp_path / "d"), compression=compression, bits=4)
    store.save(kv, b"\\x01" * 20, [3, 7], 40)
    before = kv.gather_rows(1, [3, 7], 40)
    pages, n = store.load(kv, b"\\x01" * 20)
    after = kv.gather_rows(1, pages, n)
    tol = 0.0 if compression == "NONE" else 0.2
    assert n == 40 and ((after[0] - before[0]).norm() / before[0].norm()).item() <= tol + 1e-7
    assert store.load(kv, b"\\x02" * 20) is None and store.metrics["disk_misses"] == 1


def test_device_watchdog_raises_on_stuck_event():
    """The lookahead path polls its completion event with a deadline; an event that never completes raises instead of blocking."""
    from deliverance_b200.engine.engine import Engine, EngineConfig

    class Stuck:
        def query(self):
            return False

    class Done:
        def query(self):
            return True

    eng = Engine.__new__(Engine)
    eng.config = EngineConfig(device_timeout_s=0.05)
    Engine._wait_event(eng, Done())
    with pytest.raises(RuntimeError, match="did not finish"):
        Engine._wait_event(eng, Stuck())


def test_sampler_reference_vectors():
    """core/src/test/.../TopKSamplerTest.java: candidate counts, combined top-k + top-p, uniform pick inside the nucleus, ranges."""
    from deliverance_b200.engine.sampler import candidate_limit, sample_top_k_top_p_batch
    from deliverance_b200.params import GeneratorParameters

    assert candidate_limit(64.0, 262_144) == 64 and candidate_limit(0.10, 100) == 90
    logits = torch.tensor([[5.0, 4.0, 3.0, 2.0, 1.0]])

    def pick(u, uniform):
        return int(sample_top_k_top_p_batch(logits, torch.tensor([1.0]), torch.tensor([2]), torch.tensor([0.95]), torch.tensor([uniform]),
                                            torch.tensor([u]))[0])

    assert pick(0.99, False) == 1 and pick(0.60, False) == 0 and pick(0.60, True) == 1
    for bad in (dict(uniform_top_p=0.0, top_p=0.9), dict(uniform_top_p=1.01, top_p=0.9), dict(uniform_top_p=1.0), dict(top_p=0.0), dict(top_k=0)):
        with pytest.raises(ValueError):
            GeneratorParameters(temperature=1.0, **bad).validate()
    with pytest.raises(ValueError):
        GeneratorParameters(temperature=0.0, top_p=0.9, uniform_top_p=1.0).validate()


def test_checkpoint_policies_reference_vectors():
    """The checkpoint lengths of the reference's KvBufferCachePrefixTest for all three policies."""
    from deliverance_b200.kv.paged import KvCacheSettings as S

    big = 10**6
    fb = S(block_size=4, policy="FIXED_BLOCKS", max_prefix_tokens=big)
    assert [fb.checkpoint_lengths(n) for n in (3, 4, 15)] == [[], [4], [4, 8, 12]]
    al = S(block_size=4, policy="ANCHORS_AND_LARGEST", max_prefix_tokens=1000, checkpoints=4, anchors=(4, 8, 12))
    assert al.checkpoint_lengths(35) == [4, 8, 12, 32]
    assert [al.checkpoint_lengths(n) for n in (3, 4, 15)] == [[], [4], [4, 8, 12]]
    assert S(block_size=4, policy="ANCHORS_AND_LARGEST", max_prefix_tokens=big, checkpoints=3, anchors=(4, 8, 12, 16)).checkpoint_lengths(35) == [4, 8, 32]
    assert S(block_size=32, policy="ANCHORS_AND_LARGEST", max_prefix_tokens=512, checkpoints=4).checkpoint_lengths(5000) == [32, 64, 128, 512]
    assert S(block_size=4, policy="ANCHORS_AND_LARGEST", max_prefix_tokens=16, anchors=(4, 8)).checkpoint_lengths(16) == [4, 8, 16]
    se = S(block_size=4, max_prefix_tokens=big, checkpoints=6)
    assert se.policy == "START_AND_END" and se.checkpoint_lengths(35) == [4, 8, 12, 24, 28, 32]
    assert [se.checkpoint_lengths(n) for n in (3, 4, 15)] == [[], [4], [4, 8, 12]]
    assert S(block_size=32, max_prefix_tokens=512, checkpoints=4).checkpoint_lengths(5000) == [32, 64, 480, 512]
    assert S(block_size=32, max_prefix_tokens=512, checkpoints=4).checkpoint_lengths(100) == [32, 64, 96]


@pytest.mark.parametrize("family,lookahead", [("qwen3", False), ("qwen3", "force"), ("granitemoehybrid", False)])
def test_memory_pressure_preempts_and_recomputes(tmp_path, family, lookahead):
    """Random arrivals into a page pool far too small for all of them: younger sequences are preempted (pages released,
    cache rebuilt by recompute when they are re-admitted) and every request still produces exactly the tokens of an isolated
    run, greedy and seeded sampling alike; all pages come back at the end."""
    d = str(tmp_path / "m")
    write_tiny_model(d, family, seed=11, std=0.08)
    model = DecoderModel(load_config(d), "cpu").load(WeightLoader(d))
    rng = random.Random(5)
    shared = [rng.randrange(3, 250) for _ in range(70)]
    jobs = []
    for i in range(10):
        p = (shared[: rng.choice([32, 64, 70])] if rng.random() < 0.6 else []) + [rng.randrange(3, 250) for _ in range(rng.randrange(1, 40))]
        params = GeneratorParameters(max_tokens=rng.randrange(20, 110), temperature=0.0 if i % 3 else 0.8, top_p=None if i % 3 else 0.9, seed=i)
        jobs.append((p, params, rng.randrange(0, 6)))

    def fresh(params):
        return GeneratorParameters(max_tokens=params.max_tokens, temperature=params.temperature, top_p=params.top_p, seed=params.seed)

    singles = [Engine(model, EngineConfig(num_pages=64, max_batch_tokens=64, lookahead=False), eos_ids=(-1,)).generate(p, fresh(q)).token_ids
               for p, q, _ in jobs]
    eng = Engine(model, EngineConfig(num_pages=9, max_batch_tokens=48, max_seqs=6, lookahead=lookahead, max_state_slots=8,
                                     kv=KvCacheSettings(max_prefix_tokens=4096, policy="FIXED_BLOCKS")), eos_ids=(-1,))
    reqs = [None] * len(jobs)
    step = 0
    while step < 3000 and (eng.has_work() or any(r is None for r in reqs)):
        for i, (p, q, at) in enumerate(jobs):
            if at == step:
                reqs[i] = eng.add_request(p, fresh(q))
        if eng.has_work():
            eng.step()
            eng.kv.audit([r.pages for r in eng.running])  # reference counts, holder counts and the free list stay consistent
        step += 1
    assert [r.output for r in reqs] == singles
    assert eng.metrics.get("preemptions", 0) > 0 and sum(r.preemptions for r in reqs) == eng.metrics["preemptions"]
    eng.kv.prefix.clear()
    assert eng.kv.allocator.available() == eng.kv.num_pages - 1 and not eng.running and not eng.waiting
    with pytest.raises(MemoryError):  # a single sequence that cannot fit is an error, not a hang
        small = Engine(model, EngineConfig(num_pages=3, max_batch_tokens=48, lookahead=False), eos_ids=(-1,))
        small.generate(shared[:40], GeneratorParameters(max_tokens=60))


def test_disk_store_age_sweeper_and_byte_limit(tmp_path):
    import os
    import time

    from deliverance_b200.kv.disk import DiskPrefixStore
    from deliverance_b200.kv.paged import PagedKVCache

    layout = {"layers": 2, "kv_heads": 2, "head_dim": 64, "layer_kinds": ["attention", "attention"]}
    kv = PagedKVCache(layout, 16, "cpu", torch.float32)
    store = DiskPrefixStore(str(tmp_path / "d"), compression="NONE", max_age_s=100.0)
    keys = [bytes([i]) * 20 for i in range(3)]
    for k in keys:
        store.save(kv, k, [1, 2], 40)
    old = time.time() - 1000
    os.utime(store._path(keys[0]), (old, old))
    open(os.path.join(store.dir, "dead.kv.tmp"), "w").close()
    os.utime(os.path.join(store.dir, "dead.kv.tmp"), (old, old))
    assert store.sweep() == 2 and not store.has(keys[0]) and store.has(keys[1]) and not os.path.exists(os.path.join(store.dir, "dead.kv.tmp"))
    for k in keys[1:]:
        os.utime(store._path(k), (time.time() - 90, time.time() - 90))
    assert store.load(kv, keys[1]) is not None  # a hit refreshes the time stamp
    assert store.sweep(time.time() + 50) == 1 and store.has(keys[1]) and not store.has(keys[2])
    one = os.path.getsize(store._path(keys[1]))
    small = DiskPrefixStore(str(tmp_path / "e"), compression="NONE", max_bytes=int(one * 2.5))
    for i, k in enumerate(keys + [b"\x09" * 20]):
        small.save(kv, k, [1, 2], 40)
        os.utime(small._path(k), (time.time() - 100 + i, time.time() - 100 + i))
    small._trim()
    assert [small.has(k) for k in keys + [b"\x09" * 20]] == [False, False, True, True] and small.metrics["disk_bytes"] == 2 * one


def test_reclaimable_pages_are_counted_exactly():
    """Entries of several checkpoint lengths share pages and running sequences hold cached pages too: only pages held by
    nothing but cache entries count as reclaimable, and the incremental bookkeeping survives stores, hits and evictions."""
    from deliverance_b200.kv.paged import PagedKVCache

    layout = {"layers": 1, "kv_heads": 1, "head_dim": 64, "layer_kinds": ["attention"]}
    kv = PagedKVCache(layout, 9, "cpu", torch.float32, KvCacheSettings(block_size=32, policy="FIXED_BLOCKS", max_prefix_tokens=4096))
    toks = list(range(3, 3 + 96))
    pages: list = []
    kv.ensure_pages(pages, 96)  # 3 pages; 5 stay free
    kv.prefix.store("", toks, pages)  # entries at 32, 64, 96 share the chain
    assert kv.prefix.held == {pages[0]: 3, pages[1]: 2, pages[2]: 1} and kv.prefix.reclaimable(99) == 0  # the sequence still holds them
    assert kv.can_allocate(5) and not kv.can_allocate(6)
    kv.release_pages(list(pages))
    assert kv.prefix.reclaimable(99) == 3 and kv.prefix.reclaimable(2) == 2 and kv.can_allocate(8) and not kv.can_allocate(9)
    hit = kv.prefix.lookup("", toks[:64] + [7, 7])  # a new sequence takes two of the cached pages
    assert hit.length == 64 and kv.prefix.reclaimable(99) == 1 and kv.can_allocate(6) and not kv.can_allocate(7)
    kv.release_pages(list(hit.pages))
    kv.prefix.evict_one()  # the 32-token entry (least recently used)
    assert kv.prefix.held == {pages[0]: 2, pages[1]: 2, pages[2]: 1} and kv.prefix.reclaimable(99) == 3
    kv.prefix.clear()
    assert kv.prefix.held == {} and kv.allocator.available() == 8


def test_oom_fails_one_request_and_reset_returns_every_page(tiny):
    """A sequence the pool cannot hold fails alone (the others finish); Engine.reset() after a fault returns all pages."""
    eng = _engine(tiny, pages=5, chunk=64, lookahead=False)
    eng.eos_ids = frozenset((-1,))
    small = eng.add_request([5, 6, 7], GeneratorParameters(max_tokens=4))
    big = eng.add_request(list(range(3, 120)), GeneratorParameters(max_tokens=100))  # 117 + 100 tokens > 4 pages of 32
    done = []
    while eng.has_work():
        done += eng.step()
    assert small.finish_reason == FinishReason.MAX_TOKENS and len(small.output) == 4
    assert big.finish_reason == FinishReason.ERROR and big.error.startswith("KV cache is too small") and big in done
    eng.kv.prefix.clear()
    assert eng.kv.allocator.available() == 4
    a = eng.add_request([5, 6, 7, 8], GeneratorParameters(max_tokens=50))
    b = eng.add_request([9, 10], GeneratorParameters(max_tokens=50))
    for _ in range(3):
        eng.step()
    assert eng.kv.allocator.available() < 4
    eng.reset()
    eng.kv.prefix.clear()
    assert eng.kv.allocator.available() == 4 and not eng.has_work() and a.finish_reason == FinishReason.ERROR and b.state == "finished"
    assert eng.generate([5, 6, 7], GeneratorParameters(max_tokens=3)).generated_tokens == 3  # usable afterwards


def test_prefix_cache_random_operations_keep_reference_counts_consistent():
    """Property test (hypothesis): arbitrary interleavings of sequence creation (with prefix hits), growth, caching, release and
    eviction never break the page accounting, and everything comes back at the end."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    from deliverance_b200.kv.paged import PagedKVCache

    layout = {"layers": 1, "kv_heads": 1, "head_dim": 64, "layer_kinds": ["attention"]}
    ops_strategy = st.lists(st.tuples(st.sampled_from(["new", "grow", "store", "release", "evict"]), st.integers(0, 7), st.integers(1, 90)), max_size=60)

    @settings(max_examples=60, deadline=None)
    @given(ops_strategy, st.sampled_from(["FIXED_BLOCKS", "START_AND_END", "ANCHORS_AND_LARGEST"]))
    def run(script, policy):
        kv = PagedKVCache(layout, 24, "cpu", torch.float32, KvCacheSettings(block_size=32, policy=policy, max_prefix_tokens=4096, max_entries=6))
        seqs: dict = {}
        for op, key, n in script:
            if op == "new" and key not in seqs:
                toks = [3 + (key % 3)] * 40 + [10 + key] * n  # three families of shared 40-token heads
                hit = kv.prefix.lookup("", toks)
                pages = list(hit.pages) if hit is not None else []
                try:
                    kv.ensure_pages(pages, len(toks))
                except MemoryError:
                    kv.release_pages(pages)
                    continue
                seqs[key] = (toks, pages)
            elif op == "grow" and key in seqs:
                toks, pages = seqs[key]
                toks.extend([20 + key] * n)
                try:
                    kv.ensure_pages(pages, len(toks))
                except MemoryError:
                    del toks[-n:]
            elif op == "store" and key in seqs:
                kv.prefix.store("", seqs[key][0], seqs[key][1])
            elif op == "release" and key in seqs:
                kv.release_pages(seqs.pop(key)[1])
            elif op == "evict":
                kv.prefix.evict_one()
            kv.audit([p for _, p in seqs.values()])
            assert kv.can_allocate(kv.allocator.available()) and not kv.can_allocate(kv.num_pages)
        for _, pages in seqs.values():
            kv.release_pages(pages)
        kv.prefix.clear()
        kv.audit([])
        assert kv.allocator.available() == kv.num_pages - 1

    run()


def test_decode_interleave_bounds_the_wait_of_running_sequences(tiny):
    """With decode_interleave = 1 a running sequence gets a token between the prompt chunks of later arrivals; with the default
    it waits until the whole prompt backlog is computed. Outputs are the same either way."""
    def run(k):
        eng = _engine(tiny, pages=64, chunk=16, lookahead=False, decode_interleave=k)
        eng.eos_ids = frozenset((-1,))
        first = eng.add_request([5, 6, 7], GeneratorParameters(max_tokens=12))
        while not first.output:
            eng.step()
        late = eng.add_request(list(range(3, 99)), GeneratorParameters(max_tokens=3))  # 96 tokens = 6 chunks of 16
        trace = []
        while eng.has_work():
            before = len(first.output)
            eng.step()
            trace.append("d" if len(first.output) > before else "p")
        return first.output, late.output, "".join(trace)

    a_first, a_late, a_trace = run(0)
    b_first, b_late, b_trace = run(1)
    assert a_first == b_first and a_late == b_late
    assert a_trace.startswith("pppppp") and "pp" not in b_trace and b_trace.count("p") == 6


@pytest.mark.parametrize("family", ["granitemoehybrid", "llama"])
def test_repeated_prompt_on_block_boundary_matches_uncached(tmp_path, family):
    """A prompt whose length is a multiple of the block size, sent twice: the second run may reuse cached blocks but must produce
    the tokens of an uncached run. Hybrid models must not resume a recurrent-state snapshot that already holds the last prompt
    token (that token is replayed to get logits); they take a shorter checkpoint instead."""
    d = str(tmp_path / "m")
    write_tiny_model(d, family, seed=3, std=0.08)
    model = DecoderModel(load_config(d), "cpu").load(WeightLoader(d))
    rng = random.Random(9)
    for n in (32, 64, 96, 70):
        prompt = [rng.randrange(3, 250) for _ in range(n)]

        def params():
            return GeneratorParameters(max_tokens=12, temperature=1.0, top_p=0.95, seed=n)

        want = Engine(model, EngineConfig(num_pages=64, max_batch_tokens=64, kv=KvCacheSettings(enabled=False)), eos_ids=(-1,)).generate(prompt, params())
        eng = Engine(model, EngineConfig(num_pages=64, max_batch_tokens=64), eos_ids=(-1,))
        first = eng.generate(prompt, params())
        req = eng.add_request(prompt, params())
        while eng.has_work():
            eng.step()
        assert first.token_ids == want.token_ids and req.output == want.token_ids, (family, n)
        if n >= 64:
            assert req.prefix_hit > 0, (family, n)
        if family == "granitemoehybrid":
            assert req.prefix_hit < n, (family, n)
