"""Times the UNMODIFIED reference (pure-PyTorch CPU path) on config 1 at reduced node counts.

    PYTHONDONTWRITEBYTECODE=1 python oracle/time_reference_as_is.py --ref /path/to/difflut/checkout

Run it where the reference checkout exists; the reference is a Python package that does not travel with
this repository, so the numbers it prints are recorded in the project's notes by hand and the
benchmark's `cpu_baseline` stays the oracle port.  Config 1: batch 256 x 784 features, 3-threshold
thermometer (2352 bits), RandomLayer of N six-input DWN nodes (uniform without replacement per node),
loss = sum of outputs, forward + backward.  The reference's cost is linear in the number of nodes (a Python
loop over node modules, each with an interpreted loop in its backward): the script measures two small N
and extrapolates to the configuration's 2000 nodes.
"""

import argparse
import os
import sys
import time
import warnings

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("DIFFLUT_REFERENCE"), required="DIFFLUT_REFERENCE" not in os.environ,
                    help="path of the reference checkout (or set DIFFLUT_REFERENCE)")
    ap.add_argument("--nodes", type=int, nargs="+", default=[10, 40])
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    warnings.filterwarnings("ignore")
    import difflut  # noqa: F401
    from difflut.encoder import ThermometerEncoder
    from difflut.layers import RandomLayer
    from difflut.nodes import DWNNode
    from difflut.nodes.node_config import NodeConfig

    torch.manual_seed(0)
    B = 256
    x = torch.rand(B, 784)
    enc = ThermometerEncoder(num_bits=3).fit(x)
    bits = enc.encode(x)
    rows = []
    for N in args.nodes:
        layer = RandomLayer(2352, N, DWNNode, NodeConfig(input_dim=6, output_dim=1), seed=0,
                            ensure_full_input_coverage=False)
        layer.train()
        t0 = time.perf_counter()
        out = layer(bits)
        t1 = time.perf_counter()
        out.sum().backward()
        t2 = time.perf_counter()
        rows.append((N, t1 - t0, t2 - t1))
        print(f"N={N:5d}: forward {t1 - t0:8.3f} s, backward {t2 - t1:8.3f} s", flush=True)
    (n0, f0, b0), (n1, f1, b1) = rows[0], rows[-1]
    per_node = ((f1 + b1) - (f0 + b0)) / (n1 - n0)
    fixed = (f0 + b0) - per_node * n0
    full = fixed + per_node * 2000
    print(f"per node {per_node:.4f} s, fixed {fixed:.3f} s -> extrapolated config-1 step (2000 nodes): {full:.1f} s "
          f"= {B / full:.3f} samples/s on {torch.get_num_threads()} threads (extrapolated, not measured)")


if __name__ == "__main__":
    main()
