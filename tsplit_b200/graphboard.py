"""Graph visualisation (reference ``python/graphboard/graph2fig.py:10-30``).

``show(executor, port)`` writes the executor's schedule as Graphviz DOT; when a
``dot`` binary exists it is rendered to PNG and served with ``http.server``.
Nothing here needs a display or a graphics stack."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

_server = [None]


def to_dot(executor, max_label=40):
    lines = ["digraph G {", "  rankdir=TB;", "  node [shape=box, fontsize=10];"]
    colors = {"forward": "lightblue", "backward": "lightsalmon", "update": "palegreen"}
    for n in executor.topo_order:
        label = (n.op.name if n.inputs else n.name)[:max_label]
        shape = getattr(n, "inferred_shape", None)
        if shape:
            label += "\\n" + "x".join(str(s) for s in shape)
        lines.append('  n%d [label="%s", style=filled, fillcolor=%s];' % (
            n.id, label, colors.get(n.phase, "white")))
    for n in executor.topo_order:
        for i in n.inputs:
            lines.append("  n%d -> n%d;" % (i.id, n.id))
    lines.append("}")
    return "\n".join(lines)


def show(executor, port=9997, out_dir="graphboard_out", serve=True):
    os.makedirs(out_dir, exist_ok=True)
    dot_path = os.path.join(out_dir, "output.dot")
    with open(dot_path, "w") as f:
        f.write(to_dot(executor))
    png = None
    if shutil.which("dot"):
        png = os.path.join(out_dir, "output.png")
        subprocess.run(["dot", "-Tpng", dot_path, "-o", png], check=False)
        with open(os.path.join(out_dir, "index.html"), "w") as f:
            f.write('<html><body><img src="output.png"/></body></html>')
        if serve:
            _server[0] = subprocess.Popen([sys.executable, "-m", "http.server", str(port)], cwd=out_dir,
                                          stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    return dot_path, png


def close():
    if _server[0] is not None:
        _server[0].terminate()
        _server[0] = None
