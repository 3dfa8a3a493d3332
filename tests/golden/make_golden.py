"""Generate the golden fixtures from the UNMODIFIED reference realizer.

Run in a container that holds a reference checkout:

    python oracle/build_ref.py /path/to/reference      # assembles oracle/_ref (git-ignored)
    python tests/golden/make_golden.py

For every case it (1) builds the graph twice, with the reference's own ``browsergrad_jit`` API
and with ``browsergrad_b200.graph``; (2) records the reference's post-pass graph signature
(op, input positions, shape, dtype, canonical arg) so that the restated passes and builders can
be checked without the reference; (3) realizes with the reference (``tensor.numpy()`` ->
``_realize.realize``) and stores the output; (4) checks that ``oracle/port.py`` reproduces those
bytes exactly before anything is written.  Inputs are regenerated from seeds by
``browsergrad_b200.configs`` at test time, so fixtures hold outputs and signatures only.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))

import browsergrad_jit as bg  # noqa: E402  (the reference)
from browsergrad_jit import _amp, _fusion, _ir  # noqa: E402

from browsergrad_b200 import configs, graph, passes  # noqa: E402
from oracle import port  # noqa: E402
from tests.cases import CASES, RefApi, canonical_arg, signature  # noqa: E402


def main() -> None:
    out_sig = {}
    arrays = {}
    for name, case in CASES.items():
        if not case.reference_has_it:
            print(f"{name:28s} skipped: the reference cannot build it (extension of this build)")
            continue
        inputs = case.inputs()
        # reference graph + realization
        ref_api = RefApi(bg)
        ref_t = {k: bg.from_numpy(v) for k, v in inputs.items() if not k.startswith("_")}
        ref_root_t = case.build(ref_api, ref_t, inputs)
        want = np.asarray(ref_root_t.numpy())
        ref_post = _fusion.fuse(_amp.insert_cast_pass(ref_root_t._uop))
        ref_sig = signature(_ir.toposort(ref_root_t._uop)), signature(_ir.toposort(ref_post))
        # this build's graph, passes and oracle port
        store = graph.BufferStore()
        my_t = {k: graph.from_numpy(v, store) for k, v in inputs.items() if not k.startswith("_")}
        my_root = case.build(graph, my_t, inputs)._uop
        my_post = passes.prepare(my_root)
        my_sig = signature(graph.toposort(my_root)), signature(graph.toposort(my_post))
        assert my_sig[0] == ref_sig[0], f"{name}: builder graph differs from the reference"
        assert my_sig[1] == ref_sig[1], f"{name}: post-pass graph differs from the reference"
        got = port.realize(my_post, store)
        assert got.dtype == want.dtype and got.shape == want.shape, (name, got.dtype, want.dtype)
        assert got.tobytes() == want.tobytes(), f"{name}: oracle port is not bit-identical"
        out_sig[name] = {"pre": ref_sig[0], "post": ref_sig[1]}
        arrays[name] = want
        print(f"{name:28s} ok  nodes={len(ref_sig[1])} out={want.shape} {want.dtype}")
    with open(os.path.join(HERE, "graphs.json"), "w") as fh:
        json.dump({"numpy": np.__version__, "reference_version": bg.__version__, "cases": out_sig},
                  fh, indent=0, sort_keys=True)
    np.savez_compressed(os.path.join(HERE, "outputs.npz"), **arrays)
    print("wrote", len(arrays), "cases; numpy", np.__version__)


if __name__ == "__main__":
    main()
