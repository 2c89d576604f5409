"""Make `oracle/_ref/`: the reference package in a form that can be imported anywhere.

    python oracle/make_ref.py [--reference /path/to/sparse-attention-hub]

Copies the reference's own `sparse_attention_hub/` Python package (unmodified, byte for
byte) into `oracle/_ref/sparse_attention_hub/` and writes three stand-in packages beside it
(`ray.tune`, `matplotlib`, `seaborn`) for modules the reference imports at module scope for
things off the decode path (search-space defaults, plotting).  `oracle/_ref/` is a build
output: it is listed in .gitignore and is never part of the product; `bench.py --impl
reference` and the `cpu_baseline` leg put it first on `sys.path` and time the reference's
`ResearchAttention.custom_attention` on the host cores.
"""

from __future__ import annotations

import argparse
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"

_LENIENT = '''"""Stand-in: every attribute is a callable that returns None."""


def __getattr__(name):
    if name.startswith("__"):
        raise AttributeError(name)
    return lambda *args, **kwargs: None
'''


def make(reference: Path) -> Path:
    src = reference / "sparse_attention_hub"
    if not (src / "__init__.py").exists():
        raise FileNotFoundError(f"{src} is not the reference package")
    if DEST.exists():
        shutil.rmtree(DEST)
    DEST.mkdir(parents=True)
    shutil.copytree(src, DEST / "sparse_attention_hub",
                    ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    for pkg, mods in (("ray", ["tune"]), ("matplotlib", ["pyplot"]), ("seaborn", [])):
        d = DEST / pkg
        d.mkdir()
        # bound explicitly: with the module-level __getattr__ above, `from . import x` would
        # find the catch-all callable instead of importing the sub-module
        imports = "".join(f"{m} = importlib.import_module(__name__ + '.{m}')\n" for m in mods)
        (d / "__init__.py").write_text(_LENIENT + ("\nimport importlib  # noqa: E402\n\n" + imports
                                                   if imports else ""))
        for m in mods:
            (d / f"{m}.py").write_text(_LENIENT)
    (DEST / "SOURCE.txt").write_text(f"copied from {reference} by oracle/make_ref.py; not product source\n")
    return DEST


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    args = ap.parse_args()
    print(make(Path(args.reference)))


if __name__ == "__main__":
    main()
