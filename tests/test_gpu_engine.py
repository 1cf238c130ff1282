"""The engine loop around the device forward, against the oracle driver around the oracle model:
configuration 1 (tiny Llama, 8 prompts U[32,128], 32 greedy tokens, block 16) driven exactly as
the reference's engine drives it, decode-position quirk and failing steps included. Block tables,
slot mapping, batches and sampled token ids must be bit-exact in the f32 build."""
import numpy as np
import pytest

from driver_adapters import Eng
from drivers import C1_META, c1_tensors
from oracle import driver as od

pytestmark = pytest.mark.gpu


class BlockMissing(Exception):
    pass


@pytest.fixture(scope="module")
def backend(pkg):
    if not pkg.is_available():
        pytest.fail("no CUDA device: the engine has no CPU fallback")
    return pkg.CudaBackend(0)


class Pair:
    """The oracle engine around the oracle model and the C++ engine around the device model, fed
    the same requests and stepped in lock step."""

    def __init__(self, pkg, backend, oracle, **cfg):
        weights = c1_tensors(seed=1234)
        meta = pkg.ModelMetadata(architecture="llama", name="c1", **C1_META)
        self.pkg = pkg
        self.dev = pkg.CudaTransformerModel.new(meta, weights, 160, 16, backend, compute_dtype=pkg.DType.F32,
                                                max_batch_tokens=1024, max_batch_sequences=8)
        self.ref_model = oracle.Model(num_blocks=160, block_size=16, **C1_META).load(weights)

        def ref_forward(batch):
            row = 0
            for i, n in enumerate(batch.slot_token_counts):
                if batch.positions[row + n - 1] // 16 >= len(batch.block_tables[i]):
                    raise BlockMissing()  # what both forwards report before touching the cache
                row += n
            logits = self.ref_model.forward(oracle.Batch(batch.tokens, batch.positions, batch.slot_token_counts,
                                                         batch.context_lens, batch.block_tables))
            return [oracle.argmax(r) for r in logits]

        cfg = dict(dict(max_num_seqs=8, max_num_batched_tokens=1024, max_model_len=256), **cfg)
        od.IdCounter.next = pkg.engine.next_sequence_id()
        self.ref = Eng("oracle", ref_forward, 160, 16, True, **cfg)
        self.nat = Eng("native", self.dev, 160, 16, True, **cfg)
        self.tokens = {}

    def submit(self, prompt, max_tokens):
        sid = self.ref.submit(prompt, max_tokens)
        assert sid == self.nat.submit(prompt, max_tokens)
        self.tokens[sid] = []
        return sid

    def drain(self):
        failed = 0
        for step in range(300):
            if not self.ref.has_work():
                break
            status = []
            for e, miss in ((self.ref, BlockMissing), (self.nat, self.pkg.InternalError)):
                try:
                    status.append(e.step())
                except miss:
                    status.append("failed")
            assert status[0] == status[1], f"step {step}: {status}"
            failed += status[0] == "failed"
            assert self.ref.batch() == self.nat.batch(), f"step {step}: batches differ"
            ev = self.ref.events()
            assert ev == self.nat.events(), f"step {step}: sampled tokens or completions differ"
            for x in ev:
                if x[0] == "token":
                    self.tokens[x[1]].append(x[2])
        assert not self.ref.has_work() and not self.nat.has_work()
        return failed

    def arenas_agree(self):
        kv_dev, kv_ref = self.dev.read_kv(), self.ref_model.kv().array()
        assert np.array_equal(kv_dev != 0, kv_ref != 0), "exactly the same slots were written"
        tol = self.pkg.Tolerance(self.pkg.Tolerance.F32.abs * 10, self.pkg.Tolerance.F32.rel * 10)
        rep = self.pkg.validate("kv_arena", kv_ref, kv_dev, tol)
        assert rep.passed(), rep.render()


def test_config1_through_the_engine_matches_the_oracle_driver(pkg, backend, oracle):
    oracle.set_threads(8)
    p = Pair(pkg, backend, oracle)
    rng = np.random.default_rng(7)
    prompts = [rng.integers(0, 1024, int(rng.integers(32, 129))).tolist() for _ in range(8)]
    for prompt in prompts:
        p.submit(prompt, 32)
    failed = p.drain()
    assert all(len(t) == 32 for t in p.tokens.values())
    assert failed > 0, "prompts whose length + 1 hits a block boundary fail one step in the reference"
    # a repeated prompt adopts the cached blocks of the first run and still decodes the same tokens
    first = next(iter(p.tokens.values()))
    again = p.submit(prompts[0], 32)
    p.drain()
    assert p.tokens[again] == first
    assert p.nat.sched.cache.hits() == p.ref.sched.cache.hits() > 0
    assert p.nat.sched.cache.free_blocks() == 160
    oracle.set_threads(1)
    p.arenas_agree()


def test_skipping_the_cached_prefix_keeps_the_tokens(pkg, backend, oracle):
    """The opt-in extension: sequences that adopt cached prefix blocks start their prefill after
    them. Same requests with and without it: identical generated tokens, fewer prefill tokens."""
    oracle.set_threads(8)
    rng = np.random.default_rng(11)
    shared = rng.integers(0, 1024, 64).tolist()  # four full blocks
    prompts = [shared + rng.integers(0, 1024, int(n)).tolist() for n in (9, 30, 1, 17)] + [shared, shared[:48]]
    runs = {}
    for skip in (False, True):
        p = Pair(pkg, backend, oracle, skip_cached_prefix=skip)
        first = p.submit(prompts[0], 12)
        p.drain()  # its blocks are published once its prefill has run
        for prompt in prompts[1:]:
            p.submit(prompt, 12)
        p.drain()
        stats = p.nat.sched.stats()
        assert stats == p.ref.sched.stats()
        runs[skip] = ([p.tokens[k] for k in sorted(p.tokens)], stats)
        assert first in p.tokens
        p.arenas_agree()
    oracle.set_threads(1)
    assert runs[True][0] == runs[False][0], "skipping recomputation must not change a single token"
    assert runs[False][1]["total_skipped_prefill_tokens"] == 0
    skipped = runs[True][1]["total_skipped_prefill_tokens"]
    assert skipped == 64 * 3 + 63 + 47, "three suffixed prompts, then two bare prefixes (all but their last token)"
    assert runs[True][1]["total_prefill_tokens"] == runs[False][1]["total_prefill_tokens"] - skipped


def test_logical_decode_positions_give_the_plain_greedy_decode(pkg, backend, oracle):
    """The other opt-in extension: decode tokens at position total_len - 1. No step is refused, no
    cache slot is skipped, and the tokens are those of a forward driven by hand with the same
    positions (prefill, then one token per step at its logical place)."""
    oracle.set_threads(8)
    p = Pair(pkg, backend, oracle, logical_decode_positions=True)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, 1024, n).tolist() for n in (31, 47, 16, 80)]  # 31 + 1 and 47 + 1 hit block boundaries
    ids = [p.submit(prompt, 20) for prompt in prompts]
    assert p.drain() == 0, "no refused step"
    # by hand on a fresh oracle model: contiguous tables, logical positions
    model = oracle.Model(num_blocks=160, block_size=16, **C1_META).load(c1_tensors(seed=1234))
    for sid, prompt in zip(ids, prompts):
        table = list(range(100, 100 + (len(prompt) + 20) // 16 + 1))
        logits = model.forward(oracle.Batch(prompt, list(range(len(prompt))), [len(prompt)], [len(prompt)], [table]))
        out = [oracle.argmax(logits[0])]
        for step in range(19):
            pos = len(prompt) + step
            logits = model.forward(oracle.Batch([out[-1]], [pos], [1], [pos + 1], [table]))
            out.append(oracle.argmax(logits[0]))
        assert p.tokens[sid] == out
    oracle.set_threads(1)
    p.arenas_agree()
