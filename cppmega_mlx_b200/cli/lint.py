"""``python -m cppmega_mlx_b200.cli.lint [paths…]``: run the code-base lint (``runtime/lint.py``) and print one line per finding;
exit code 1 when there is any.  Without paths it checks the package, ``bench.py`` and ``__graft_entry__.py``."""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    from ..runtime.lint import lint_paths
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("paths", nargs="*")
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    paths = args.paths or [p for p in (os.path.join(root, "cppmega_mlx_b200"), os.path.join(root, "bench.py"),
                                       os.path.join(root, "__graft_entry__.py")) if os.path.exists(p)]
    found = lint_paths(paths)
    if args.json:
        print(json.dumps({"status": "ok" if not found else "violations", "count": len(found),
                          "violations": [{"path": v.path, "line": v.line, "rule": v.rule, "message": v.message} for v in found]}))
    else:
        for v in found:
            print(v)
        print(f"{len(found)} finding(s) in {len(paths)} path(s)")
    return 1 if found else 0


if __name__ == "__main__":
    sys.exit(main())
