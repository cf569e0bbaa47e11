"""Multi-replica host logic on CPU ranks (gloo, world size 2 and 3): batch
sharding, output gather in batch order, rebasing of detection image ids.  The
compute stand-in on each rank is the numpy oracle (a softmax) -- what is under
test is the slicing and gathering, which is identical for GPU replicas."""
import os
import socket
import sys

import numpy as np
import pytest

from conftest import ROOT, pkg

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


def test_shard_bounds_cover_the_batch():
    sh = pkg("sharding")
    for total in (0, 1, 7, 64, 256):
        for world in (1, 2, 3, 8):
            spans = [sh.shard_bounds(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
                assert e0 == b1 and b0 <= e0
            assert all(e - b <= -(-total // world) if world else True for b, e in spans)


def test_rebase_detection_rows():
    sh = pkg("sharding")
    rows = np.array([[0, 3, 0.9, 0, 0, 1, 1], [1, 5, 0.8, 0, 0, 1, 1]], np.float32)
    out = sh.rebase_detection_rows(rows, 32)
    assert out[:, 0].tolist() == [32.0, 33.0] and rows[:, 0].tolist() == [0.0, 1.0]
    assert sh.rebase_detection_rows(np.zeros((0, 7), np.float32), 5).shape == (0, 7)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import importlib
    sh = importlib.import_module("mini-caffe_b200.sharding")
    oracle = importlib.import_module("oracle.numpy_oracle")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)
        logits = rng.standard_normal((7, 10)).astype(np.float32)     # 7 images: ragged shards

        def make_replica(batch):
            def run(inputs):
                assert inputs["fc"].shape[0] == batch
                return oracle.softmax(inputs["fc"], axis=1)
            return run

        dense = sh.run_sharded(make_replica, {"fc": logits}, dist=dist)

        def make_detector(batch):
            def run(inputs):
                # one row per local image: (local image id, label, score, box)
                return np.stack([[i, 1, float(inputs["fc"][i, 0]), 0, 0, 1, 1] for i in range(batch)]).astype(np.float32)
            return run

        rows = sh.run_sharded(make_detector, {"fc": logits}, dist=dist, detection=True)

        def make_sparse_detector(batch):
            def run(inputs):
                # images with a positive first logit have one detection; a replica without any emits
                # the layer's placeholder rows (label -1), one per image of its slice
                hits = [[i, 2, float(inputs["fc"][i, 0]), 0, 0, 1, 1] for i in range(batch) if inputs["fc"][i, 0] > cut]
                if hits:
                    return np.asarray(hits, np.float32)
                return np.asarray([[i, -1, -1, -1, -1, -1, -1] for i in range(batch)], np.float32)
            return run

        cut = float(np.sort(logits[:, 0])[-2])     # only the largest first logit passes: one replica has a hit
        sparse = sh.run_sharded(make_sparse_detector, {"fc": logits}, dist=dist, detection=True)
        cut = 1e9                                   # nobody has a hit: the placeholders of all images survive
        empty = sh.run_sharded(make_sparse_detector, {"fc": logits}, dist=dist, detection=True)

        def make_proposals(batch):
            def run(inputs):
                # two rois per local image, column 0 = image index within the slice
                return np.asarray([[i, 0, 0, 4 + j, 4 + j] for i in range(batch) for j in range(2)], np.float32)
            return run

        rois = sh.run_sharded(make_proposals, {"fc": logits}, dist=dist, proposal=True)
        ragged = sh.gather_rows(np.full((rank + 1, 5), rank, np.float32), dist=dist)
        if rank == 0:
            np.savez(os.path.join(tmpdir, "out.npz"), dense=dense, rows=rows, ragged=ragged, logits=logits,
                     sparse=sparse, empty=empty, rois=rois)
        else:
            assert dense is None and rows is None and ragged is None and sparse is None and rois is None
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_run_matches_single_replica(tmp_path, world):
    oracle = __import__("importlib").import_module("oracle.numpy_oracle")
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = np.load(os.path.join(str(tmp_path), "out.npz"))
    want = oracle.softmax(got["logits"], axis=1)
    assert np.array_equal(got["dense"], want)                      # batch order preserved
    assert got["rows"][:, 0].tolist() == [float(i) for i in range(7)]  # image ids rebased
    assert np.array_equal(got["rows"][:, 2], got["logits"][:, 0])
    # one replica had a detection, the others only placeholders: the single real row survives, with
    # its global image id
    best = int(np.argmax(got["logits"][:, 0]))
    assert got["sparse"].shape == (1, 7) and got["sparse"][0, 0] == best and got["sparse"][0, 1] == 2
    # no replica had any: one placeholder row per image of the whole batch, ids 0..6
    assert got["empty"].shape == (7, 7) and (got["empty"][:, 1] == -1).all()
    assert got["empty"][:, 0].tolist() == [float(i) for i in range(7)]
    # Proposal rois: image ids rebased by the slice offsets
    assert got["rois"][:, 0].tolist() == [float(i) for i in range(7) for _ in range(2)]
    assert got["ragged"].shape == (sum(r + 1 for r in range(world)), 5)
    assert got["ragged"][:, 0].tolist() == [float(r) for r in range(world) for _ in range(r + 1)]
