"""Recipe for oracle/_ref/: the reference's own torch-eager module, extracted where it lies.

TEST INFRASTRUCTURE ONLY. Run by __graft_entry__.build() on a machine that has the
reference checkout; writes oracle/_ref/eager_reference.py, which is NOT tracked (the
reference's sources are never committed here) but travels with the working tree, so that
bench.py's CPU legs can time the reference's own EagerGatedMLP class
(src/triton_gated_mlp/gated_mlp.py:73-98 with its activation table :27-37) instead of the
restatement in gated_mlp_oracle.py. The extract is made with `ast`, by node, from the file
as it is: the class EagerGatedMLP and the module-level names it uses (ACT_FWD), plus the
torch imports. Nothing of the reference's Triton path is touched or imported.
"""
from __future__ import annotations

import ast
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref" / "eager_reference.py"
WANTED_ASSIGN = {"ACT_FWD"}
WANTED_CLASS = {"EagerGatedMLP"}


def extract(reference_root: Path) -> Path | None:
    src_path = reference_root / "src" / "triton_gated_mlp" / "gated_mlp.py"
    if not src_path.exists():
        return None
    text = src_path.read_text()
    tree = ast.parse(text)
    parts = []
    for node in tree.body:
        keep = False
        if isinstance(node, ast.Assign):
            keep = any(isinstance(t, ast.Name) and t.id in WANTED_ASSIGN for t in node.targets)
        elif isinstance(node, ast.ClassDef):
            keep = node.name in WANTED_CLASS
        if keep:
            parts.append(ast.get_source_segment(text, node))
    if len(parts) != len(WANTED_ASSIGN) + len(WANTED_CLASS):
        return None
    OUT.parent.mkdir(parents=True, exist_ok=True)
    (OUT.parent / "__init__.py").write_text("")
    header = (f'"""Extracted by oracle/make_ref.py from {src_path.relative_to(reference_root)} of the reference '
              'checkout; not tracked."""\n'
              "from torch import nn\nimport torch\n\n\n")
    OUT.write_text(header + "\n\n\n".join(parts) + "\n")
    return OUT


def main() -> int:
    root = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("GMLP_REFERENCE_ROOT", "/root/reference"))
    out = extract(root)
    print(out if out else f"no reference checkout at {root}: nothing extracted")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
