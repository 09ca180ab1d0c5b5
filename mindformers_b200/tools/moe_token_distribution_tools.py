"""Charts and statistics of how tokens spread over the experts of every MoE layer during a run.

Reference: ``mindformers/tools/moe_token_distribution_tools.py`` (collects the per-step ``.npy`` dumps of each MoE
layer, merges them in step order and draws one chart per layer). Input here is the same kind of dump —
``<dir>/layer-<L>-step<N>.npy`` with one count (or load fraction) per expert, written by
``TopkBiasBalanceCallback(dump_dir=...)`` — or arrays handed over directly. Output per layer: the merged
``[steps, experts]`` table as CSV, balance statistics, and a heat-map chart. The chart is written as a self-contained
SVG (no plotting library is needed); with matplotlib installed a PNG is written as well.

    python -m mindformers_b200.tools.moe_token_distribution_tools --num_layers 4 --hot_expert_num 2 \
        --npy_files_load_path output/expert_load --save_path_prefix output/expert_load/charts
"""
from __future__ import annotations

import argparse
import json
import os
import re
from typing import Dict, List, Optional

import numpy as np

_NAME_RE = re.compile(r"layer-(\d+)-step(\d+)\.npy$")


def collect_npy_files(path: str) -> Dict[int, List[str]]:
    """``{layer: [files in step order]}`` of every ``layer-L-stepN.npy`` below ``path``."""
    found: Dict[int, List[tuple]] = {}
    for root, _, files in os.walk(path):
        for f in files:
            m = _NAME_RE.search(f)
            if m:
                found.setdefault(int(m.group(1)), []).append((int(m.group(2)), os.path.join(root, f)))
    return {layer: [p for _, p in sorted(items)] for layer, items in sorted(found.items())}


def merge_npy_files(files: List[str]) -> np.ndarray:
    """Step-ordered dumps of one layer → ``[steps, experts]`` (a dump that already holds several steps is kept)."""
    rows = []
    for f in files:
        a = np.asarray(np.load(f), dtype=np.float64)
        rows.append(a.reshape(-1, a.shape[-1]))
    if not rows:
        raise FileNotFoundError("no dumps for this layer")
    return np.concatenate(rows, axis=0)


def distribution_stats(table: np.ndarray, hot_expert_num: int = 1) -> dict:
    """Balance figures of a ``[steps, experts]`` table: per-step max / mean load ratio and coefficient of variation,
    the experts that are hottest / coldest over the run, and the share of tokens that the hottest ones take."""
    table = np.asarray(table, dtype=np.float64)
    total = table.sum(axis=1, keepdims=True)
    frac = np.divide(table, total, out=np.zeros_like(table), where=total > 0)
    mean = frac.mean(axis=1)
    imbalance = np.divide(frac.max(axis=1), mean, out=np.ones_like(mean), where=mean > 0)
    cv = np.divide(frac.std(axis=1), mean, out=np.zeros_like(mean), where=mean > 0)
    overall = frac.mean(axis=0)
    order = np.argsort(-overall)
    k = max(1, min(int(hot_expert_num), table.shape[1]))
    return {"steps": int(table.shape[0]), "experts": int(table.shape[1]),
            "max_over_mean": {"first": float(imbalance[0]), "last": float(imbalance[-1]), "worst": float(imbalance.max())},
            "coefficient_of_variation": {"first": float(cv[0]), "last": float(cv[-1]), "mean": float(cv.mean())},
            "hot_experts": [int(e) for e in order[:k]], "cold_experts": [int(e) for e in order[::-1][:k]],
            "hot_share": float(overall[order[:k]].sum()), "idle_experts": [int(e) for e in np.where(overall == 0)[0]]}


def _color(v: float) -> str:
    """White (0) → dark blue (1)."""
    v = min(max(v, 0.0), 1.0)
    r, g, b = int(255 - 215 * v), int(255 - 160 * v), int(255 - 60 * v)
    return f"#{r:02x}{g:02x}{b:02x}"


def heatmap_svg(table: np.ndarray, title: str, max_cells: int = 400) -> str:
    """SVG heat map: one column per step (steps are averaged into at most ``max_cells`` columns), one row per expert,
    colour = share of the step's tokens relative to the largest share in the chart."""
    table = np.asarray(table, dtype=np.float64)
    total = table.sum(axis=1, keepdims=True)
    frac = np.divide(table, total, out=np.zeros_like(table), where=total > 0)
    steps, experts = frac.shape
    if steps > max_cells:
        edges = np.linspace(0, steps, max_cells + 1).astype(int)
        frac = np.stack([frac[a:b].mean(axis=0) for a, b in zip(edges[:-1], edges[1:]) if b > a])
    cols = frac.shape[0]
    cw = max(2.0, min(12.0, 900.0 / cols))
    ch = max(3.0, min(16.0, 480.0 / experts))
    left, top = 60, 34
    width, height = left + cols * cw + 20, top + experts * ch + 40
    peak = frac.max() or 1.0
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width:.0f}" height="{height:.0f}" font-family="sans-serif" font-size="11">',
           f'<text x="{left}" y="16" font-size="13">{title}: share of tokens per expert (rows) over steps (columns), '
           f'darkest = {peak:.3f}</text>']
    for c in range(cols):
        for e in range(experts):
            out.append(f'<rect x="{left + c * cw:.1f}" y="{top + e * ch:.1f}" width="{cw:.1f}" height="{ch:.1f}" '
                       f'fill="{_color(frac[c, e] / peak)}"/>')
    for e in range(0, experts, max(1, experts // 16)):
        out.append(f'<text x="{left - 6}" y="{top + e * ch + ch * 0.8:.1f}" text-anchor="end">{e}</text>')
    out.append(f'<text x="{left}" y="{height - 12:.0f}">step 0</text>')
    out.append(f'<text x="{left + cols * cw:.0f}" y="{height - 12:.0f}" text-anchor="end">step {steps - 1}</text>')
    out.append("</svg>")
    return "\n".join(out)


def write_layer_report(layer: int, table: np.ndarray, save_path_prefix: str, hot_expert_num: int = 1) -> dict:
    os.makedirs(os.path.dirname(save_path_prefix) or ".", exist_ok=True)
    base = f"{save_path_prefix}layer-{layer}"
    np.savetxt(base + ".csv", table, delimiter=",", fmt="%.6g")
    stats = distribution_stats(table, hot_expert_num)
    with open(base + ".json", "w") as f:
        json.dump(stats, f, indent=1)
    with open(base + ".svg", "w") as f:
        f.write(heatmap_svg(table, f"MoE layer {layer}"))
    try:                                        # optional raster chart
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        total = table.sum(axis=1, keepdims=True)
        plt.figure(figsize=(10, 4))
        plt.imshow((table / np.maximum(total, 1e-12)).T, aspect="auto", cmap="Blues")
        plt.xlabel("step")
        plt.ylabel("expert")
        plt.title(f"MoE layer {layer}")
        plt.colorbar()
        plt.savefig(base + ".png", dpi=120)
        plt.close()
    except ImportError:
        pass
    return stats


def generate_reports(npy_files_load_path: str, save_path_prefix: str, num_layers: Optional[int] = None,
                     hot_expert_num: int = 1) -> Dict[int, dict]:
    files = collect_npy_files(npy_files_load_path)
    if not files:
        raise FileNotFoundError(f"no layer-L-stepN.npy dumps under {npy_files_load_path}")
    layers = sorted(files) if num_layers is None else [l for l in sorted(files) if l < num_layers]
    return {l: write_layer_report(l, merge_npy_files(files[l]), save_path_prefix, hot_expert_num) for l in layers}


def main(argv=None):
    ap = argparse.ArgumentParser(description="merge expert-load dumps and draw one chart per MoE layer")
    ap.add_argument("--num_layers", type=int, default=None, help="only layers below this index")
    ap.add_argument("--hot_expert_num", type=int, default=1, help="how many hottest / coldest experts to list")
    ap.add_argument("--npy_files_load_path", required=True)
    ap.add_argument("--save_path_prefix", default="./token_distribution/")
    a = ap.parse_args(argv)
    for layer, stats in generate_reports(a.npy_files_load_path, a.save_path_prefix, a.num_layers, a.hot_expert_num).items():
        print(f"layer {layer}: {stats['steps']} steps, max/mean load {stats['max_over_mean']['last']:.2f} "
              f"(worst {stats['max_over_mean']['worst']:.2f}), hot experts {stats['hot_experts']}, "
              f"idle {stats['idle_experts']}")


if __name__ == "__main__":
    main()
