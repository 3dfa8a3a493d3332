"""Assemble the reference's own Python realizer as an importable package under ``oracle/_ref``.

TEST INFRASTRUCTURE, not product code.  The reference ships ``browsergrad_jit`` as Python
sources that its TypeScript host writes into a Pyodide file system
(packages/browsergrad-jit/src/install.ts:6-20); its ``__init__.py`` only exists as a
template string inside packages/browsergrad-jit/src/python/index.ts:59-749.  This script
links the sources from where they lie in a reference checkout and renders that template,
so the unmodified reference realizer can be imported under CPython to validate the NumPy
restatement in ``oracle/port.py`` and to generate ``tests/golden`` vectors.

The output directory is git-ignored: nothing of the reference enters the history.
Usage: ``python oracle/build_ref.py [reference_checkout]``.
"""
from __future__ import annotations

import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def build(reference_root: str) -> str:
    src = os.path.join(reference_root, "packages", "browsergrad-jit", "src", "python")
    if not os.path.isdir(src):
        raise FileNotFoundError(f"no browsergrad-jit python sources under {reference_root}")
    pkg_dir = os.path.join(OUT, "browsergrad_jit")
    if os.path.isdir(pkg_dir):
        shutil.rmtree(pkg_dir)
    os.makedirs(pkg_dir)
    for name in sorted(os.listdir(src)):
        if (name.startswith("_") and name.endswith(".py")) or name.endswith(".v1.json"):
            shutil.copyfile(os.path.join(src, name), os.path.join(pkg_dir, name))
    with open(os.path.join(reference_root, "packages", "browsergrad-jit", "package.json")) as fh:
        version = json.load(fh)["version"]
    with open(os.path.join(src, "index.ts"), encoding="utf-8") as fh:
        ts = fh.read()
    start = ts.index("const INIT_PY = `") + len("const INIT_PY = `")
    end = ts.index("`;\n\nexport interface PythonSource", start)
    body = ts[start:end]
    # Undo the template-literal escaping: \` -> `, \\ -> \, ${pkg.version} -> version.
    body = body.replace("\\`", "`").replace("${pkg.version}", version).replace("\\\\", "\\")
    body = body.replace("\\${", "${")
    with open(os.path.join(pkg_dir, "__init__.py"), "w", encoding="utf-8") as fh:
        fh.write(body)
    return pkg_dir


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BG_REFERENCE_ROOT", "/root/reference")
    print(build(root))
