"""Checkpoint round trips: ModelOpt NVFP4 tensors, sharded load, generation equality."""
import torch

from hibana_b200.engine.executor import Executor
from hibana_b200.engine.request import SamplingParams
from hibana_b200.models.dense import DenseModel
from hibana_b200.target import dense_tiny, scaled
from hibana_b200.weights import checkpoint, modelopt


def test_dense_checkpoint_roundtrip_and_tp_shards(tmp_path):
    t = scaled(dense_tiny(), weight_format="nvfp4")
    model = DenseModel(t, "cpu", seed=0)
    for lin in model.linears():
        lin.set_input_amax(4.0)
    checkpoint.save_dense(model, str(tmp_path), layers_per_file=1)
    loaded = checkpoint.load_dense(t, str(tmp_path))
    for a, b in zip(model.linears(), loaded.linears()):
        assert torch.equal(a.wq.q, b.wq.q) and torch.equal(a.wq.sf, b.wq.sf) and torch.equal(a.alpha, b.alpha)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, t.vocab, (20,), generator=g).tolist() for _ in range(2)]
    sp = SamplingParams(max_tokens=5)
    a = [r.output_ids for r in Executor(model, max_batch=2, max_ctx=64, use_graphs=False).generate_batch(prompts, sp)]
    b = [r.output_ids for r in Executor(loaded, max_batch=2, max_ctx=64, use_graphs=False).generate_batch(prompts, sp)]
    assert a == b
    # a tensor-parallel shard read from the file equals the shard cut from the in-memory model
    ref = DenseModel.sharded(t, 2, 1, "cpu", seed=0)
    shard = checkpoint.load_dense(t, str(tmp_path), tp=2, rank=1)
    for x, y in zip(ref.linears(), shard.linears()):
        assert torch.equal(x.wq.q, y.wq.q) and torch.equal(x.wq.sf, y.wq.sf)


def test_unpack_fp4():
    q = torch.tensor([[0x21, 0xF7]], dtype=torch.uint8)
    assert modelopt.unpack_fp4(q).tolist() == [[0.5, 1.0, 6.0, -6.0]]
