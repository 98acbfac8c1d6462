"""Writes ``torch_op_schemas.json``: the operator schemas the reference registers under
``torch.ops.mxfp6`` (csrc/torch_extension.cu TORCH_LIBRARY block, csrc/moe.cu
TORCH_LIBRARY_FRAGMENT block), in the dispatcher's canonical spelling.

Run where the reference's sources are present:
    python tests/golden/make_torch_op_schemas.py <reference root>
Only the ``m.def("...")`` string literals are read; nothing is compiled or imported.
"""

from __future__ import annotations

import json
import re
import sys
from pathlib import Path

import torch


def schemas_of(path: Path) -> dict[str, str]:
    text = path.read_text()
    found = {}
    for match in re.finditer(r"m\.def\(\s*((?:\"(?:[^\"\\]|\\.)*\"\s*)+)\)", text):
        schema = "".join(re.findall(r"\"((?:[^\"\\]|\\.)*)\"", match.group(1)))
        parsed = torch._C.parse_schema(schema)
        found[parsed.name] = str(parsed)
    return found


def main() -> None:
    root = Path(sys.argv[1])
    schemas = {}
    for relative in ("csrc/torch_extension.cu", "csrc/moe.cu"):
        schemas.update(schemas_of(root / relative))
    out = Path(__file__).with_name("torch_op_schemas.json")
    out.write_text(json.dumps(schemas, indent=1, sort_keys=True) + "\n")
    print(f"{len(schemas)} schemas -> {out}")


if __name__ == "__main__":
    main()
