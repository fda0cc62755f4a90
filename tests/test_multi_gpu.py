"""Two ranks on two GPUs (one process each): sharded batch, NCCL all-reduce of the flat gradient buffer inside
gn_train_batch, identical Adam on both ranks.  The first step's loss, every gradient tensor and the post-step
weights must equal the full-batch CPU checker step at the strict tolerance, the second step must follow, and the
two replicas must stay bit-identical.  Skipped on a box with fewer than two GPUs."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CASES = [("mlp", {}, 64, 1), ("transformer_small", dict(vocab=512, dim=64, seq_len=16, heads=4, ff_dim=128, n_blocks=2), 8, 1),
         ("transformer_large", dict(vocab=500, dim=128, seq_len=256, heads=2, ff_dim=256, n_blocks=1), 4, 1),      # tcgen05 attention on each shard
         ("transformer_small", dict(vocab=300, dim=48, seq_len=20, heads=3, ff_dim=100, n_blocks=1), 8, 4),        # four reference workers over two ranks
         ("cnn", dict(hw=12, c0=2, c1=5, c2=7, classes=3), 10, 1),
         ("lstm", dict(in_size=5, hidden=24, seq_len=7), 12, 1),       # one worker chunk spans both ranks: update factors gathered, scan replicated
         ("lstm", dict(in_size=5, hidden=24, seq_len=7), 12, 4),       # worker chunks inside the ranks' shards
         ("cnn_bn", dict(hw=10, c0=2, c1=5, classes=3), 8, 1),         # BatchNorm2D running statistics across ranks
         ("gru", dict(in_size=5, hidden=24, seq_len=7), 10, 1)]


def _rank(rank, world, uid, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from goneuron_b200 import configs
    from goneuron_b200.sequential import Adam, Device, Sequential
    from goneuron_b200.sharding import shard_bounds
    dev = Device(rank, rank, world, uid)
    for ci, (name, kw, gb, W) in enumerate(CASES):
        layers, loss_kind, params, x, y, lr = configs.make_case(name, batch=gb, **kw)
        s, e = shard_bounds(gb, rank, world)
        model = Sequential(layers, dev, virtual_workers=W).Compile(Adam(lr), loss_kind)
        model.SetParams(params)
        loss1 = model.TrainBatch(x[s:e], y[s:e], gb, s)
        grads1, params1 = model.Gradients(), model.Params()
        loss2 = model.TrainBatch(x[s:e], y[s:e], gb, s)
        np.savez(os.path.join(out_dir, f"r{rank}_c{ci}.npz"), grads1=grads1, params1=params1, grads=model.Gradients(), params=model.Params(),
                 losses=np.array([loss1, loss2]), state=model.State(), ar_ms=model.stats().allreduce_ms)
        model.Close()
    dev.close()


def test_two_gpu_data_parallel_step(tmp_path, oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from goneuron_b200 import configs
    from goneuron_b200.sequential import Device
    from tests.parity import TOL, assert_grads_close, assert_weights_close, norm_err
    uid = Device.unique_id()
    mp.spawn(_rank, args=(2, uid, str(tmp_path)), nprocs=2, join=True)
    for ci, (name, kw, gb, W) in enumerate(CASES):
        layers, loss_kind, params, x, y, lr = configs.make_case(name, batch=gb, **kw)
        ref = oracle.OracleState(layers, loss_kind, params, lr=lr)
        l1 = ref.train_batch(x, y, W=W, threads=8, precision=64)
        g1, p1 = ref.grads.copy(), ref.params.copy()
        lit = oracle.OracleState(layers, loss_kind, params, lr=lr)
        lit.train_batch(x, y, W=W, threads=1 if W == 1 else W, precision=32)
        l2 = ref.train_batch(x, y, W=W, threads=8, precision=64)
        r0, r1 = (np.load(tmp_path / f"r{r}_c{ci}.npz") for r in (0, 1))
        # the replicas never diverge: gradients, weights and running statistics are bit-identical on both ranks
        for key in ("grads1", "params1", "grads", "params", "state"):
            assert np.array_equal(r0[key], r1[key]), (name, key)
        # first step: strict tolerance on the loss, every gradient tensor and the post-step weights
        assert abs(r0["losses"][0] - l1) <= TOL * max(1.0, abs(l1)), (name, r0["losses"][0], l1)
        worst = assert_grads_close(layers, r0["grads1"], g1, floor=lit.grads)
        assert_weights_close(r0["params1"], p1, params, g1, lr)
        print(f"2 GPUs, {name} batch {gb} W {W}: loss {r0['losses'][0]:.6f} (cpu {l1:.6f}); worst gradient tensor {worst[1]} at {worst[2]:.2e}")
        # second step: the Adam update of the first one has amplified fp32 noise, so a looser bound
        assert abs(r0["losses"][1] - l2) <= TOL * max(1.0, abs(l2))
        assert norm_err(r0["grads"], ref.grads) <= 2e-3
        if ref.state.size:
            assert norm_err(r0["state"], ref.state) <= TOL
