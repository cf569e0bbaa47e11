"""Batch sharding across replicas and the final output gather.

The engine scales like the reference's multi-device use (one thread or process
per GPU, each with its own Net and a full copy of the weights --
mini-caffe tests/run_net.cpp:222-246): every layer on the hot path is
independent along the batch axis, so a global batch is cut into contiguous
slices, each replica runs its slice with no communication, and only the final
outputs are gathered.  There is no collective inside the forward pass.

  dense outputs (class scores)      concatenated in batch order
  DetectionOutput rows              concatenated in image order, column 0 (the
                                    image index within the replica's slice)
                                    rebased by the slice offset.  A replica
                                    without any detection emits one placeholder
                                    row per image (label -1), as the reference
                                    does for a whole batch without detections
                                    (src/layers/detection_output_layer.cpp:171-188);
                                    placeholders are dropped unless no replica
                                    has a real row, so that the gathered result
                                    is what one device would have produced
  Proposal rois                     concatenated; column 0 (the image index
                                    within the replica's slice, for the batched
                                    layer) rebased by the slice offset
"""
import numpy as np


def shard_bounds(total, world, rank):
    """[begin, end) of the contiguous slice of `total` items owned by `rank`:
    ceil(total / world) items per replica, the last ones may get fewer or none."""
    per = -(-total // world)
    begin = min(total, rank * per)
    return begin, min(total, begin + per)


def rebase_detection_rows(rows, image_offset):
    """Rows [image, label, score, xmin, ymin, xmax, ymax] of a replica -> global image ids."""
    rows = np.array(rows, dtype=np.float32, copy=True)
    if rows.size:
        rows[:, 0] += np.float32(image_offset)
    return rows


def rebase_proposal_rows(rois, image_offset):
    """Rows [image, x1, y1, x2, y2] of a replica's batched Proposal layer -> global image ids."""
    return rebase_detection_rows(rois, image_offset)


def merge_detection_rows(parts):
    """Rows of all replicas (already rebased), in replica order -> rows of the whole batch: real rows
    only, or, when there is none at all, the placeholder rows (label -1) of every image."""
    parts = [np.asarray(p, dtype=np.float32).reshape(-1, 7) for p in parts if p is not None and np.size(p)]
    if not parts:
        return np.zeros((0, 7), dtype=np.float32)
    rows = np.concatenate(parts, axis=0)
    real = rows[:, 1] != -1
    return rows[real] if real.any() else rows


def gather_rows(local_rows, dist=None, dst=0):
    """Concatenate ragged [R_i, C] float arrays of all ranks on `dst` in rank order
    (None elsewhere).  With dist=None the local array is returned."""
    local_rows = np.ascontiguousarray(local_rows, dtype=np.float32)
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return local_rows
    world, rank = dist.get_world_size(), dist.get_rank()
    gathered = [None] * world if rank == dst else None
    dist.gather_object(local_rows, gathered, dst=dst)
    if rank != dst:
        return None
    cols = max(g.shape[1] for g in gathered)
    parts = [g for g in gathered if g.shape[0] > 0]
    return np.concatenate(parts, axis=0) if parts else np.zeros((0, cols), dtype=np.float32)


def run_sharded(make_replica, global_inputs, dist=None, detection=False, proposal=False):
    """Run `make_replica(batch)` -> callable(inputs) -> ndarray on this rank's slice of
    `global_inputs` (dict name -> array with the batch on axis 0) and gather on rank 0.
    detection / proposal: the output is DetectionOutput rows / Proposal rois (see above)."""
    world = dist.get_world_size() if dist is not None and dist.is_initialized() else 1
    rank = dist.get_rank() if world > 1 else 0
    total = next(iter(global_inputs.values())).shape[0]
    begin, end = shard_bounds(total, world, rank)
    if end > begin:
        local = {k: v[begin:end] for k, v in global_inputs.items()}
        out = make_replica(end - begin)(local)
        if detection or proposal:
            out = rebase_detection_rows(out, begin)
    else:
        out = None
    if world == 1:
        return merge_detection_rows([out]) if detection and out is not None else out
    payload = out if out is not None else np.zeros((0, 0), dtype=np.float32)
    gathered = [None] * world if rank == 0 else None
    dist.gather_object(payload, gathered, dst=0)
    if rank != 0:
        return None
    parts = [g for g in gathered if g.size]
    if detection:
        return merge_detection_rows(parts)
    return np.concatenate(parts, axis=0)
