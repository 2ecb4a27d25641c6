"""Renders and compiles the reference's own layer-1 CUDA plugin for the medium structure.

TEST INFRASTRUCTURE ONLY.  The reference generates its layer-1 kernels from an execution contract
(symmetrix/source/symmetrix/jit_codegen.py: render_jit_r1_cuda_plugin, :3420-3454); its pure-Python
generator imports without the native extension.  This script runs that generator in place (nothing of
it is copied into the repository) on the contract fixture of the OMAT-0 / MPA-0 medium structure
(symmetrix/test/data/execution_contracts/jit_r1_mace_mpa0_medium_contract.json), compiles the rendered
source for sm_100a and leaves, under oracle/_ref/ (git-ignored; it travels with a repository snapshot):
    libsymmetrix_ref_r1_cuda.so          the reference's plugin (symmetrix_jit_cuda_plugin_query_v2)
    r1_medium_coupling.json              the contract's sparse coupling terms (row, output, coefficient)
Usage:  python oracle/build_reference_r1_plugin.py <reference checkout>   (oracle/Makefile passes its REFERENCE_ROOT)
"""
from __future__ import annotations

import importlib
import json
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main():
    given = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT")
    if not given:
        raise SystemExit("usage: build_reference_r1_plugin.py <reference checkout>   (or set REFERENCE_ROOT)")
    root = Path(given)
    out = HERE / "_ref"
    if not root.exists():
        print("reference checkout not present: keeping prebuilt oracle/_ref (if any)")
        return
    out.mkdir(exist_ok=True)
    sys.path.insert(0, str(root / "symmetrix" / "source"))
    codegen = importlib.import_module("symmetrix.jit_codegen")
    contract_path = root / "symmetrix" / "test" / "data" / "execution_contracts" / "jit_r1_mace_mpa0_medium_contract.json"
    contract = json.loads(contract_path.read_text())
    target = out / "libsymmetrix_ref_r1_cuda.so"
    source = out / "r1_medium_plugin.cu"
    source.write_text(codegen.render_jit_r1_cuda_plugin(contract, 100))
    subprocess.run([os.environ.get("NVCC", "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler",
                    "-fPIC", "-shared", "-o", str(target), str(source)], check=True)
    source.unlink()          # the rendered source is the reference's code: only the binary is kept
    terms = [{"row": t["row"], "output": t["lme"], "coefficient": t["coefficient"]} for t in contract["sparse_coupling"]["terms"]]
    (out / "r1_medium_coupling.json").write_text(json.dumps({"channels": contract["channels"], "terms": terms}))
    print("built", target)


if __name__ == "__main__":
    main()
