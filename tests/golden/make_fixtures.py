"""Generates tests/golden/fixtures/<case>.npz by running each case of cases.py on the
reference's own CPU transformer.  Run in a container that has the reference tree:

    python tests/golden/make_fixtures.py [/path/to/ngraph-python] [case ...]

Without a path the tree named by B200NG_REFERENCE, else oracle/_ref/ (oracle/make_ref.py), is
used.  The reference is imported unmodified (ngraph_python_b200/ngraph_compat supplies what it needs).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def main(ref_root, only=None):
    from oracle import ref_env
    if ref_root:
        os.environ["B200NG_REFERENCE"] = ref_root
    if ref_env.install() is None:
        raise SystemExit("no reference tree: pass its path or run oracle/make_ref.py")
    import ngraph as ng
    import ngraph.transformers as ngt
    from tests.golden import cases
    out_dir = os.path.join(HERE, "fixtures")
    os.makedirs(out_dir, exist_ok=True)
    for name, build in sorted(cases.CASES.items()):
        if only and name not in only:
            continue
        outs, params, vals = build(ng)
        t = ngt.make_transformer_factory("cpu")()
        comp = t.computation(outs, *params)
        data = {}      # inputs are not stored: cases.py regenerates them from its seeds
        for rep in range(cases.REPEAT.get(name, 1)):
            res = comp(*vals)
            for k, r in enumerate(res):
                data["out%d_%d" % (rep, k)] = np.array(r, copy=True)
        t.close()
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **data)
        print(name, {k: v.shape for k, v in data.items() if k.startswith("out")})


if __name__ == "__main__":
    argv = sys.argv[1:]
    root = argv.pop(0) if argv and os.path.isdir(argv[0]) else None
    main(root, set(argv))
