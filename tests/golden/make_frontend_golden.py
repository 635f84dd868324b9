"""Regenerates tests/golden/suite_frontend.json: what this repository's .tca frontend makes of the reference's
own suite kernels (testing/kernels/*/*.tca of a tcacomp checkout).

    python tests/golden/make_frontend_golden.py /path/to/tcacomp

For every kernel the file records what tcab_module_kernel_describe reports -- operator class, canonical lambda
texts, init, capture names, reduced axis or operand layout, tensor and scalar parameter names -- never the
kernel source. The parity tests run these plans on the device against the oracle's restatement of the
reference's runners, which ties the reference's kernel TEXT to the numbers the runners expect."""
import glob
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def derive(checkout: str) -> dict:
    from tcacomp_b200 import tca
    out = {}
    for path in sorted(glob.glob(os.path.join(checkout, "testing", "kernels", "*", "*.tca"))):
        module = tca.Module(open(path).read())
        assert len(module.names()) == 1, path
        name = module.names()[0]
        entry = module.describe(name)
        entry["launcher"] = name
        out[os.path.splitext(os.path.basename(path))[0]] = entry
    return out


if __name__ == "__main__":
    from oracle.build import REF_DEFAULT
    checkout = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TCAB_REFERENCE", REF_DEFAULT)
    golden = derive(checkout)
    with open(os.path.join(ROOT, "tests", "golden", "suite_frontend.json"), "w") as f:
        json.dump(golden, f, indent=1, sort_keys=True)
        f.write("\n")
    print(f"{len(golden)} kernels")
