"""Batch sharding and the gradient allreduce on CPU ranks (gloo, world size 2): host-side logic only."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sphmap.parallel import GradReducer, shard_batch


def test_shard_batch_covers_the_batch_evenly():
    for B in (1, 7, 64):
        for world in (1, 2, 3, 8):
            parts = [shard_batch(B, r, world) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == B
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
            sizes = [hi - lo for lo, hi in parts]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # each rank owns a slice of the batch and produces its partial dW / dBias = sum over its images
    B = 6
    per_image_gw = torch.arange(B * 12, dtype=torch.float32).view(B, 3, 2, 2)
    per_image_gb = torch.arange(B * 3, dtype=torch.float32).view(B, 3)
    lo, hi = shard_batch(B, rank, world)
    red = GradReducer()
    layers = []
    for scale in (1.0, 2.0):       # two "layers", submitted one after the other, finished together
        gw, gb = per_image_gw[lo:hi].sum(0) * scale, per_image_gb[lo:hi].sum(0) * scale
        red.submit(gw, gb)
        layers.append((gw, gb, scale))
    red.finish()
    ok = all(torch.equal(gw, per_image_gw.sum(0) * s) and torch.equal(gb, per_image_gb.sum(0) * s) for gw, gb, s in layers)
    # the same through the reducer's own buffers: the flat allocation behind (gw, gb) is reduced where it lies
    gw, gb = red.buffers((3, 2, 2), (3,), torch.float32, "cpu")
    for scale in (1.0, 3.0):       # the buffers are reused from step to step
        gw.copy_(per_image_gw[lo:hi].sum(0) * scale)
        gb.copy_(per_image_gb[lo:hi].sum(0) * scale)
        red.submit(gw, gb)
        packed = red.pending[-1][1]
        red.finish()
        ok = ok and packed is None and torch.equal(gw, per_image_gw.sum(0) * scale) and torch.equal(gb, per_image_gb.sum(0) * scale)
    # several layers in one arena: per layer (mode "layer") or as one message at the end of backward (mode "step")
    for mode in ("layer", "step"):
        red2 = GradReducer(mode=mode)
        pairs = red2.arena([((3, 2, 2), (3,)), ((3, 2, 2), (3,))], torch.float32, "cpu")
        for (gw, gb), scale in zip(pairs, (1.0, 2.0)):
            gw.copy_(per_image_gw[lo:hi].sum(0) * scale)
            gb.copy_(per_image_gb[lo:hi].sum(0) * scale)
            red2.submit(gw, gb)
        ok = ok and len(red2.pending) == (2 if mode == "layer" else 0)
        red2.finish()
        for (gw, gb), scale in zip(pairs, (1.0, 2.0)):
            ok = ok and torch.equal(gw, per_image_gw.sum(0) * scale) and torch.equal(gb, per_image_gb.sum(0) * scale)
    out[rank] = bool(ok)
    dist.destroy_process_group()


def test_grad_reducer_sums_across_two_gloo_ranks():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_grad_reducer_is_a_no_op_without_a_process_group():
    red = GradReducer()
    gw, gb = torch.ones(2, 2), torch.ones(2)
    red.submit(gw, gb)
    red.finish()
    assert not red.enabled and torch.equal(gw, torch.ones(2, 2))


def test_grad_reducer_buffers_are_adjacent_views_of_one_allocation():
    gw, gb = GradReducer().buffers((4, 3, 9), (4,), torch.float32, "cpu")
    assert gw.shape == (4, 3, 9) and gb.shape == (4,) and gw.is_contiguous() and gb.is_contiguous()
    assert gb.data_ptr() == gw.data_ptr() + gw.numel() * 4
    pairs = GradReducer().arena([((4, 3, 9), (4,)), ((5, 4, 9), (5,))], torch.float32, "cpu")
    for (gw, gb), (ws, bs) in zip(pairs, (((4, 3, 9), (4,)), ((5, 4, 9), (5,)))):
        assert gw.shape == ws and gb.shape == bs and gb.data_ptr() == gw.data_ptr() + gw.numel() * 4
        assert (gw.data_ptr() - pairs[0][0].data_ptr()) % 256 == 0
