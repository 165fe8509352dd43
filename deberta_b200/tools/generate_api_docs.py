"""Docstrings → Markdown API reference.

Usage::

    python -m deberta_b200.tools.generate_api_docs [--out docs/api] [--check]

Walks the package's modules with ``ast`` (nothing is imported, so it runs without torch or a GPU), groups them into
pages (``data.md``, ``modeling.md``, ``training.md`` as the reference's ``tools/generate_api_docs.py`` does, plus
``ops.md``, ``parallel.md``, ``kernels.md``), and writes one section per module with its public classes, methods and
functions: signature line and docstring. ``kernels.md`` is generated from the comments of ``csrc/kernels.h``.
``--check`` writes nothing and exits 1 when a page on disk differs from what would be generated.
"""

from __future__ import annotations

import argparse
import ast
import re
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parents[1]
REPO = PKG.parent

PAGES: dict[str, tuple[str, list[str]]] = {
    "config.md": ("Configuration and CLI", ["config.py", "cli.py", "export_cli.py", "run_layout.py"]),
    "data.md": ("Data pipeline", ["data/loading.py", "data/streaming.py", "data/collator.py", "data/synthetic.py"]),
    "modeling.md": ("Models", ["models/deberta_v2.py", "models/rope.py", "models/rope_encoder.py", "models/norm.py",
                               "models/rtd.py", "models/builder.py", "models/export_utils.py", "models/mask_utils.py",
                               "models/activations.py"]),
    "ops.md": ("Operators", ["ops/gemm.py", "ops/linear.py", "ops/norm.py", "ops/attention.py", "ops/attention_cuda.py",
                             "ops/heads.py", "ops/heads_cuda.py", "ops/microbench.py", "ops/_lib.py", "build.py"]),
    "parallel.md": ("Parallel runtime", ["parallel/dist.py", "parallel/engine.py", "parallel/peer.py",
                                         "parallel/comm_selftest.py"]),
    "training.md": ("Training", ["training/entrypoint.py", "training/trainer.py", "training/runtime.py",
                                 "training/loop_utils.py", "training/schedulers.py", "training/checkpointing.py",
                                 "training/run_management.py", "training/run_config.py", "training/metrics.py",
                                 "training/tracker_utils.py", "training/export_helpers.py", "training/watchdog.py",
                                 "utils/checkpoint.py"]),
    "tools.md": ("Tools", ["tools/audit_contracts.py", "tools/kernel_drift_probe.py", "tools/generate_api_docs.py"]),
}


def _signature(node: ast.FunctionDef | ast.AsyncFunctionDef) -> str:
    try:
        args = ast.unparse(node.args)
    except Exception:  # noqa: BLE001
        args = "..."
    ret = f" -> {ast.unparse(node.returns)}" if node.returns is not None else ""
    return f"{node.name}({args}){ret}"


def _doc(node: ast.AST) -> str:
    d = ast.get_docstring(node, clean=True)
    return d.strip() if d else ""


def _public(name: str) -> bool:
    return not name.startswith("_") or name in ("__init__", "__call__")


def render_module(rel: str) -> str:
    path = PKG / rel
    if not path.exists():
        return ""
    tree = ast.parse(path.read_text())
    mod = "deberta_b200." + rel[:-3].replace("/", ".")
    out = [f"## `{mod}`", ""]
    if _doc(tree):
        out += [_doc(tree), ""]
    for node in tree.body:
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)) and _public(node.name) and node.name != "__init__":
            out += [f"### `{_signature(node)}`", ""]
            if _doc(node):
                out += [_doc(node), ""]
        elif isinstance(node, ast.ClassDef) and _public(node.name):
            bases = ", ".join(ast.unparse(b) for b in node.bases)
            out += [f"### class `{node.name}`" + (f"(`{bases}`)" if bases else ""), ""]
            if _doc(node):
                out += [_doc(node), ""]
            for sub in node.body:
                if isinstance(sub, (ast.FunctionDef, ast.AsyncFunctionDef)) and _public(sub.name) and _doc(sub):
                    out += [f"- `{_signature(sub)}` — {_doc(sub).splitlines()[0]}"]
            out.append("")
    return "\n".join(out).rstrip() + "\n"


def render_kernels() -> str:
    """One entry per C entry point of ``csrc/kernels.h`` with the comment block that precedes it."""
    text = (PKG / "csrc" / "kernels.h").read_text() + "\n" + (PKG / "csrc" / "no_alloc.h").read_text()
    out = ["# Kernel library (C ABI)", "",
           "Entry points of `deberta_b200/_native/libdb200_kernels.so` (sources under `deberta_b200/csrc`). All take a "
           "`cudaStream_t` as their last argument, return 0 on success and a negative code for rejected arguments, and "
           "never allocate device memory unless stated.", ""]
    lines = text.splitlines()
    comment: list[str] = []
    i = 0
    while i < len(lines):
        line = lines[i]
        if line.strip().startswith("//"):
            comment.append(line.strip().lstrip("/ ").rstrip())
        elif re.match(r"^\s*(int|void|const char\*|int\*)\s+\*?db200_\w+\s*\(", line):
            code, _, trailing = line.partition("//")
            decl = code.strip()
            if trailing.strip():
                comment.append(trailing.strip())
            while not decl.rstrip().endswith(";") and i + 1 < len(lines):
                i += 1
                code, _, trailing = lines[i].partition("//")
                decl += " " + code.strip()
                if trailing.strip():
                    comment.append(trailing.strip())
            name = re.search(r"(db200_\w+)", decl).group(1)
            out += [f"## `{name}`", "", "```c", decl, "```", ""]
            if comment:
                out += [" ".join(comment), ""]
            comment = []
        elif line.strip():
            if not line.strip().startswith(("typedef", "}", "#", "const", "void*", "int ", "long", "float", "unsigned", "struct")):
                comment = []
        i += 1
    return "\n".join(out).rstrip() + "\n"


def build_pages() -> dict[str, str]:
    pages = {}
    for fname, (title, modules) in PAGES.items():
        body = [f"# {title}", "", "Generated by `python -m deberta_b200.tools.generate_api_docs`; edit the docstrings, not this file.", ""]
        body += [render_module(m) for m in modules]
        pages[fname] = "\n".join(b for b in body if b is not None)
    pages["kernels.md"] = render_kernels()
    return pages


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", default=str(REPO / "docs" / "api"))
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args(argv)
    out = Path(args.out)
    pages = build_pages()
    stale = []
    for name, text in pages.items():
        target = out / name
        if args.check:
            if not target.exists() or target.read_text() != text:
                stale.append(name)
        else:
            out.mkdir(parents=True, exist_ok=True)
            target.write_text(text)
    if args.check:
        if stale:
            print("stale API pages: " + ", ".join(stale))
            return 1
        print("API pages are up to date")
        return 0
    print(f"wrote {len(pages)} pages to {out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
