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


def test_config1_through_the_engine_matches_the_oracle_driver(pkg, backend, oracle):
    weights = c1_tensors(seed=1234)
    meta = pkg.ModelMetadata(architecture="llama", name="c1", **C1_META)
    dev = pkg.CudaTransformerModel.new(meta, weights, 160, 16, backend, compute_dtype=pkg.DType.F32,
                                       max_batch_tokens=1024, max_batch_sequences=8)
    ref_model = oracle.Model(num_blocks=160, block_size=16, **C1_META).load(weights)
    oracle.set_threads(8)

    def ref_forward(batch):
        row = 0
        for i, n in enumerate(batch.slot_token_counts):
            if batch.positions[row + n - 1] // 16 >= len(batch.block_tables[i]):
                raise BlockMissing()  # what both forwards report before touching the cache
            row += n
        logits = ref_model.forward(oracle.Batch(batch.tokens, batch.positions, batch.slot_token_counts,
                                                batch.context_lens, batch.block_tables))
        return [oracle.argmax(r) for r in logits]

    cfg = dict(max_num_seqs=8, max_num_batched_tokens=1024, max_model_len=256)
    od.IdCounter.next = pkg.engine.next_sequence_id()
    ref = Eng("oracle", ref_forward, 160, 16, True, **cfg)
    nat = Eng("native", dev, 160, 16, True, **cfg)
    rng = np.random.default_rng(7)
    prompts = [rng.integers(0, 1024, int(rng.integers(32, 129))).tolist() for _ in range(8)]
    for p in prompts:
        assert ref.submit(p, 32) == nat.submit(p, 32)

    def drain():
        failed = tokens = 0
        for step in range(200):
            if not ref.has_work():
                break
            status = []
            for e, miss in ((ref, BlockMissing), (nat, pkg.InternalError)):
                try:
                    status.append(e.step())
                except miss:
                    status.append("failed")
            assert status[0] == status[1], f"step {step}: {status}"
            failed += status[0] == "failed"
            assert ref.batch() == nat.batch(), f"step {step}: batches differ"
            ev = ref.events()
            assert ev == nat.events(), f"step {step}: sampled tokens or completions differ"
            tokens += sum(1 for x in ev if x[0] == "token")
        assert not ref.has_work() and not nat.has_work()
        return failed, tokens

    failed, tokens = drain()
    assert tokens == 8 * 32
    assert failed > 0, "prompts whose length + 1 hits a block boundary fail one step in the reference"
    # a repeated prompt adopts the cached blocks of the first run and still decodes the same tokens
    assert ref.submit(prompts[0], 32) == nat.submit(prompts[0], 32)
    drain()
    assert nat.sched.cache.hits() == ref.sched.cache.hits() > 0
    assert nat.sched.cache.free_blocks() == 160
    oracle.set_threads(1)
    kv_dev, kv_ref = dev.read_kv(), ref_model.kv().array()
    assert np.array_equal(kv_dev != 0, kv_ref != 0), "exactly the same slots were written"
    rep = pkg.validate("kv_arena", kv_ref, kv_dev, pkg.Tolerance(pkg.Tolerance.F32.abs * 10, pkg.Tolerance.F32.rel * 10))
    assert rep.passed(), rep.render()
