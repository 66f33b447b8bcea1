"""Sweep results as tables (role of zoology/analysis/utils.py ``fetch_wandb_runs`` and the plotting examples in
zoology/analysis/mqar_plotting_example.py): runs are read from what the trainer writes locally — the results CSV
(one row per finished run) and the JSON-lines logs of ``ZOOLOGY_LOG_DIR`` (one file per run with its config and
per-epoch metrics) — there is no network on the training box to fetch anything from. The MQAR figure of the reference
(accuracy against model dimension, one panel per sequence length, one line per mixer, best learning rate per point) is
produced as a pivot table, and optionally as a matplotlib figure when that library is importable.
"""
from __future__ import annotations

import glob
import json
import os

import pandas as pd


def load_results(csv_path: str | None = None, log_dir: str | None = None) -> pd.DataFrame:
    """One row per run. ``csv_path``: the trainer's results CSV. ``log_dir``: JSON-lines run logs; the best
    ``valid/accuracy`` of each log and the fields of its config are flattened into the row."""
    frames = []
    if csv_path and os.path.exists(csv_path):
        frames.append(pd.read_csv(csv_path))
    if log_dir:
        rows = []
        for path in sorted(glob.glob(os.path.join(log_dir, "*.jsonl"))):
            cfg, best, n_params, state = {}, None, None, None
            with open(path) as f:
                for line in f:
                    d = json.loads(line)
                    if "config" in d:
                        cfg = d["config"]
                    n_params = d.get("num_parameters", n_params)
                    state = d.get("state_size", state)
                    if "valid/accuracy" in d and (best is None or d["valid/accuracy"] > best["valid/accuracy"]):
                        best = d
            if best is None:
                continue
            model, data = cfg.get("model", {}), cfg.get("data", {})
            mixer = (model.get("sequence_mixer") or {}).get("name", "")
            train_cfgs = data.get("train_configs") or [{}]
            rows.append({"run_id": cfg.get("run_id", os.path.basename(path)[:-6]), "mixer": mixer, "model": model.get("name"), "d_model": model.get("d_model"),
                         "n_layers": model.get("n_layers"), "vocab_size": model.get("vocab_size"), "seq_len": train_cfgs[0].get("input_seq_len"),
                         "lr": cfg.get("learning_rate"), "n_params": n_params, "state_size": state, "best_acc": best["valid/accuracy"],
                         "best_loss": best.get("valid/loss"), "best_epoch": best.get("epoch")})
        if rows:
            frames.append(pd.DataFrame(rows))
    if not frames:
        return pd.DataFrame(columns=["run_id", "mixer", "d_model", "seq_len", "lr", "best_acc"])
    df = pd.concat(frames, ignore_index=True)
    return df.drop_duplicates(subset=["run_id"], keep="last") if "run_id" in df else df


def short_mixer(name: str) -> str:
    return str(name).rsplit(".", 1)[-1]


def best_by(df: pd.DataFrame, keys=("mixer", "seq_len", "d_model"), metric: str = "best_acc") -> pd.DataFrame:
    """Best run of every ``keys`` group (the reference keeps the best learning rate per plotted point)."""
    if df.empty:
        return df
    idx = df.groupby(list(keys))[metric].idxmax()
    return df.loc[idx].reset_index(drop=True)


def mqar_table(df: pd.DataFrame, metric: str = "best_acc") -> pd.DataFrame:
    """Rows (seq_len, mixer), columns d_model, values the best ``metric`` over learning rates."""
    if df.empty:
        return df
    d = best_by(df.assign(mixer=df["mixer"].map(short_mixer)), metric=metric)
    return d.pivot_table(index=["seq_len", "mixer"], columns="d_model", values=metric, aggfunc="max").sort_index()


PALETTE = ["#222222", "#59A14F", "#4E79A7", "#E15759", "#F28E2B", "#76B7B2", "#9C755F", "#EDC948", "#B07AA1", "#BAB0AC", "#D3722C"]


def _svg_panels(d: pd.DataFrame, lens, metric: str, path: str) -> None:
    """Dependency-free figure: the same panels as the matplotlib one, written as SVG (log2 x axis, y from 0 to 1 or to
    the data's maximum)."""
    import math
    W, H, L, R, T, B = 300, 230, 46, 10, 26, 36
    mixers = sorted(d["mixer"].unique())
    color = {m: PALETTE[i % len(PALETTE)] for i, m in enumerate(mixers)}
    xs = sorted(d["d_model"].unique())
    lx = [math.log2(x) for x in xs]
    x0, x1 = min(lx) - 0.2, max(lx) + 0.2
    ymax = max(1.0, float(d[metric].max()))
    px = lambda v: L + (math.log2(v) - x0) / max(x1 - x0, 1e-9) * (W - L - R)
    py = lambda v: T + (1 - v / ymax) * (H - T - B)
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W * len(lens)}" height="{H + 16 * ((len(mixers) + 3) // 4)}" font-family="sans-serif" font-size="10">',
           '<rect width="100%" height="100%" fill="white"/>']
    for i, sl in enumerate(lens):
        ox = i * W
        out.append(f'<g transform="translate({ox},0)"><text x="{W / 2}" y="14" text-anchor="middle" font-size="11">seq_len {sl}</text>')
        out.append(f'<rect x="{L}" y="{T}" width="{W - L - R}" height="{H - T - B}" fill="none" stroke="#888"/>')
        for k in range(5):
            v = ymax * k / 4
            out.append(f'<line x1="{L}" x2="{W - R}" y1="{py(v):.1f}" y2="{py(v):.1f}" stroke="#ddd"/><text x="{L - 4}" y="{py(v) + 3:.1f}" text-anchor="end">{v:.2f}</text>')
        for x in xs:
            out.append(f'<text x="{px(x):.1f}" y="{H - B + 12}" text-anchor="middle">{x}</text>')
        out.append(f'<text x="{W / 2}" y="{H - 6}" text-anchor="middle">d_model</text>')
        for m, g in d[d["seq_len"] == sl].groupby("mixer"):
            g = g.sort_values("d_model")
            pts = " ".join(f"{px(a):.1f},{py(b):.1f}" for a, b in zip(g["d_model"], g[metric]))
            out.append(f'<polyline points="{pts}" fill="none" stroke="{color[m]}" stroke-width="1.5"/>')
            out += [f'<circle cx="{px(a):.1f}" cy="{py(b):.1f}" r="2.5" fill="{color[m]}"/>' for a, b in zip(g["d_model"], g[metric])]
        out.append("</g>")
    for j, m in enumerate(mixers):
        x, y = 10 + (j % 4) * 150, H + 12 + 16 * (j // 4)
        out.append(f'<rect x="{x}" y="{y - 8}" width="10" height="10" fill="{color[m]}"/><text x="{x + 14}" y="{y + 1}">{m}</text>')
    out.append("</svg>")
    with open(path, "w") as f:
        f.write("\n".join(out))


def plot_mqar(df: pd.DataFrame, path: str, metric: str = "best_acc") -> bool:
    """One panel per sequence length, accuracy against d_model, one line per mixer (the figure of the reference's
    zoology/analysis/mqar_plotting_example.py). With matplotlib the file type follows the extension; without it, or for
    a ``.svg`` path, a plain SVG is written. Always returns True once the file exists."""
    d = best_by(df.assign(mixer=df["mixer"].map(short_mixer)), metric=metric)
    lens = sorted(d["seq_len"].unique())
    try:
        if path.endswith(".svg"):
            raise ImportError
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        _svg_panels(d, lens, metric, path if path.endswith(".svg") else path + ".svg")
        return True
    fig, axes = plt.subplots(1, len(lens), figsize=(4 * len(lens), 3.2), squeeze=False)
    for ax, L in zip(axes[0], lens):
        for mixer, g in d[d["seq_len"] == L].groupby("mixer"):
            g = g.sort_values("d_model")
            ax.plot(g["d_model"], g[metric], marker="o", label=mixer)
        ax.set_xscale("log", base=2)
        ax.set_title(f"seq_len {L}")
        ax.set_xlabel("d_model")
        ax.set_ylabel(metric)
    axes[0][0].legend(fontsize=7)
    fig.tight_layout()
    fig.savefig(path, dpi=120)
    plt.close(fig)
    return True


def state_tradeoff_table(df: pd.DataFrame, metric: str = "best_acc", family: str = "model") -> pd.DataFrame:
    """Recall against memory (the figure of zoology/experiments/paper_configs/arxiv24_based_figure2/plot.py): per model
    family and recurrent-state size the best ``metric`` over learning rates, plus ``on_frontier``: no run of the same
    family reaches at least this accuracy with a smaller state."""
    need = {family, "state_size", metric}
    if df.empty or not need <= set(df.columns):
        return pd.DataFrame(columns=[family, "state_size", metric, "on_frontier"])
    d = df.dropna(subset=["state_size", metric]).copy()
    d[family] = d[family].fillna(d["mixer"].map(short_mixer)) if "mixer" in d else d[family]
    d = d.groupby([family, "state_size"], as_index=False)[metric].max().sort_values([family, "state_size"])
    best_so_far = d.groupby(family)[metric].cummax()
    prev_best = best_so_far.groupby(d[family]).shift(1)
    d["on_frontier"] = prev_best.isna() | (d[metric] > prev_best)
    return d.reset_index(drop=True)


def plot_state_tradeoff(df: pd.DataFrame, path: str, metric: str = "best_acc", family: str = "model") -> bool:
    """Scatter of every (family, state size) point with the family's frontier as a line; SVG, log2 x axis."""
    import math
    t = state_tradeoff_table(df, metric, family)
    if t.empty:
        return False
    W, H, L, R, T, B = 520, 340, 52, 130, 20, 40
    fams = sorted(t[family].unique())
    color = {m: PALETTE[i % len(PALETTE)] for i, m in enumerate(fams)}
    lx = [math.log2(max(float(v), 1.0)) for v in t["state_size"]]
    x0, x1 = min(lx) - 0.3, max(lx) + 0.3
    ymax = max(1.0, float(t[metric].max()))
    px = lambda v: L + (math.log2(max(float(v), 1.0)) - x0) / max(x1 - x0, 1e-9) * (W - L - R)
    py = lambda v: T + (1 - v / ymax) * (H - T - B)
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" font-family="sans-serif" font-size="10">',
           '<rect width="100%" height="100%" fill="white"/>', f'<rect x="{L}" y="{T}" width="{W - L - R}" height="{H - T - B}" fill="none" stroke="#888"/>']
    for k in range(5):
        v = ymax * k / 4
        out.append(f'<line x1="{L}" x2="{W - R}" y1="{py(v):.1f}" y2="{py(v):.1f}" stroke="#ddd"/><text x="{L - 4}" y="{py(v) + 3:.1f}" text-anchor="end">{v:.2f}</text>')
    for e in range(int(math.ceil(x0)), int(math.floor(x1)) + 1, max(1, int((x1 - x0) // 8) or 1)):
        out.append(f'<text x="{px(2 ** e):.1f}" y="{H - B + 12}" text-anchor="middle">2^{e}</text>')
    out.append(f'<text x="{(L + W - R) / 2}" y="{H - 8}" text-anchor="middle">recurrent state size (elements)</text>')
    for j, m in enumerate(fams):
        g = t[t[family] == m]
        out += [f'<circle cx="{px(a):.1f}" cy="{py(b):.1f}" r="2.5" fill="{color[m]}" fill-opacity="0.55"/>' for a, b in zip(g["state_size"], g[metric])]
        f_ = g[g["on_frontier"]]
        if len(f_) > 1:
            pts = " ".join(f"{px(a):.1f},{py(b):.1f}" for a, b in zip(f_["state_size"], f_[metric]))
            out.append(f'<polyline points="{pts}" fill="none" stroke="{color[m]}" stroke-width="1.5"/>')
        out.append(f'<rect x="{W - R + 10}" y="{T + 14 * j}" width="10" height="10" fill="{color[m]}"/><text x="{W - R + 24}" y="{T + 9 + 14 * j}">{m}</text>')
    out.append("</svg>")
    with open(path if path.endswith(".svg") else path + ".svg", "w") as f:
        f.write("\n".join(out))
    return True


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--csv", default=os.environ.get("ZOOLOGY_CSV", "zoology_results.csv"))
    ap.add_argument("--log-dir", default=os.environ.get("ZOOLOGY_LOG_DIR"))
    ap.add_argument("--plot", default=None, help="write the figure to this file")
    ap.add_argument("--figure", choices=["mqar", "tradeoff"], default="mqar",
                    help="mqar: accuracy against width per sequence length; tradeoff: accuracy against recurrent-state size per family")
    a = ap.parse_args(argv)
    df = load_results(a.csv, a.log_dir)
    table = mqar_table(df) if a.figure == "mqar" else state_tradeoff_table(df)
    print(table.to_string() if not table.empty else "no runs found")
    if a.plot and not df.empty:
        (plot_mqar if a.figure == "mqar" else plot_state_tradeoff)(df, a.plot)
        print("figure written")
    return table


if __name__ == "__main__":
    main()
