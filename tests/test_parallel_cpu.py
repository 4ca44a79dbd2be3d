"""Host logic of the batch-sharded path on CPU ranks (gloo, world size 2)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cs2d import ops, parallel
from cs2d.synthetic import make_inputs
from oracle import cs2d_oracle as O


def test_shard_bounds_cover_batch():
    for batch in (1, 5, 32, 33):
        for world in (1, 2, 3, 8):
            spans = [parallel.shard_bounds(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
    with pytest.raises(ValueError):
        parallel.shard_bounds(4, 2, 2)


def test_param_grad_layout_and_unpack():
    total, parts = ops.param_grad_layout(6, 4, True, False, True)
    assert total == 24 + 6 + 1 and parts["dA"] == (0, 24) and parts["dD"] == (24, 6) and parts["dA_decay"] == (30, 1)
    flat = torch.arange(total, dtype=torch.float32)
    dA, dD, dbias, ddecay = parallel.unpack_param_grads(flat, 6, 4, True, False, True)
    assert dA.shape == (6, 4) and dbias is None and float(ddecay) == 30.0 and dD[0] == 24.0
    total, _ = ops.param_grad_layout(6, 4, False, True, False)
    dA, dD, dbias, _ = parallel.unpack_param_grads(torch.ones(total), 6, 4, False, True, False, delta_dim=3)
    assert dD is None and dbias.shape == (3,) and float(dbias[0]) == 2.0


def _rank_main(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        inp = make_inputs(4, 2, 3, 4, 6, 9, seed=0)
        lo, hi = parallel.shard_bounds(4, rank, world)
        sl = {k: (v[lo:hi] if k in ("u", "delta", "B", "C", "dout") else v) for k, v in inp.items()}
        # the CPU oracle stands in for the kernel: this test is about sharding + the one collective
        g = O.bwd(sl["u"], sl["delta"], sl["A"], sl["B"], sl["C"], sl["D"], sl["delta_bias"], sl["dout"], True)
        total, parts = ops.param_grad_layout(6, 4, True, True, False)
        flat = torch.zeros(total)
        for name in ("dA", "dD", "ddelta_bias"):
            off, n = parts[name]
            flat[off:off + n] = torch.from_numpy(np.asarray(g[name], dtype=np.float32).reshape(-1))
        parallel.allreduce_param_grads(flat)
        np.save(os.path.join(tmp, f"flat{rank}.npy"), flat.numpy())
        np.save(os.path.join(tmp, f"du{rank}.npy"), g["du"])
    finally:
        dist.destroy_process_group()


def test_two_ranks_match_single_process(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    inp = make_inputs(4, 2, 3, 4, 6, 9, seed=0)
    g = O.bwd(inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"], inp["delta_bias"], inp["dout"], True)
    f0, f1 = (np.load(tmp_path / f"flat{r}.npy") for r in (0, 1))
    np.testing.assert_array_equal(f0, f1)
    dA, dD, dbias, _ = parallel.unpack_param_grads(torch.from_numpy(f0), 6, 4, True, True, False)
    np.testing.assert_allclose(dA.numpy(), g["dA"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(dD.numpy(), g["dD"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(dbias.numpy(), g["ddelta_bias"], rtol=1e-5, atol=1e-5)
    du = np.concatenate([np.load(tmp_path / f"du{r}.npy") for r in (0, 1)], 0)
    np.testing.assert_allclose(du, g["du"], rtol=1e-12, atol=1e-12)


def test_allreduce_is_a_noop_without_a_process_group():
    flat = torch.ones(4)
    assert parallel.allreduce_param_grads(flat) is None and float(flat.sum()) == 4.0
