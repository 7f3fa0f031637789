"""Writes tests/golden/kernel_offsets.json by running the reference's own
generate_kernel_offsets (minuet/utils/helpers.py:165-212, pure numpy).

The reference package cannot be imported as a whole without its compiled
extension, so helpers.py is loaded alone with a stub parent package.  Run once
in a container that has the reference checked out:

    python tests/golden/make_offsets_golden.py /path/to/reference
"""
import importlib.util
import json
import os
import sys
import types


def load_reference_helpers(root):
    pkg = types.ModuleType("minuet")
    pkg.__path__ = [os.path.join(root, "minuet")]
    utils = types.ModuleType("minuet.utils")
    utils.__path__ = [os.path.join(root, "minuet", "utils")]
    sys.modules.setdefault("minuet", pkg)
    sys.modules.setdefault("minuet.utils", utils)
    for name in ("typing", "helpers"):
        path = os.path.join(root, "minuet", "utils", name + ".py")
        spec = importlib.util.spec_from_file_location("minuet.utils." + name, path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules["minuet.utils." + name] = mod
        spec.loader.exec_module(mod)
    return sys.modules["minuet.utils.helpers"]


def main():
    root = sys.argv[1]
    helpers = load_reference_helpers(root)
    cases = []
    for layout in ("minuet", "minkowski", "torchsparse"):
        for ndim, ks, ss, dil in [(3, 3, 1, 1), (3, 2, 1, 1), (3, 3, 2, 1), (3, 2, 2, 1),
                                  (3, 3, 1, 2), (3, (3, 1, 2), (1, 2, 4), (2, 1, 1)),
                                  (3, 5, 1, 1), (2, 3, 1, 1), (2, (2, 3), 2, 1), (1, 3, 4, 1),
                                  (4, 2, 1, 1), (4, (1, 3, 1, 2), 1, 1)]:
            table = helpers.generate_kernel_offsets(ndim=ndim, kernel_size=ks, source_stride=ss,
                                                    dilation=dil, layout=layout)
            cases.append({"layout": layout, "ndim": ndim, "kernel_size": ks, "source_stride": ss,
                          "dilation": dil, "offsets": table.tolist()})
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernel_offsets.json")
    with open(out, "w") as f:
        json.dump({"source": "minuet/utils/helpers.py generate_kernel_offsets", "cases": cases}, f)
    print(out, len(cases))


if __name__ == "__main__":
    main()
