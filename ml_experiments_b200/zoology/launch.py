"""Sweep launcher: ``python -m ml_experiments_b200.zoology.launch sweep.py [-p] [--gpus 0,1,...]``.

The Python file must define ``configs: list[TrainConfig]``. Sequentially by default; with ``-p`` one worker process
per visible GPU pulls configs from a shared queue (the reference schedules one Ray task per config with
``num_gpus=1``, zoology/launch.py:48-81; here a process pool pinned with ``CUDA_VISIBLE_DEVICES`` does the same without
a cluster runtime). A failing config is reported and does not stop the sweep.
"""
from __future__ import annotations

import argparse
import importlib.util
import multiprocessing as mp
import os
import traceback
from datetime import datetime


def load_configs(python_file: str) -> list:
    # sweep files written for the reference import ``zoology.config`` / ``zoology.data...``: serve those names from this
    # package (a real ``zoology`` installation, if there is one, keeps precedence)
    from ..compat import install
    install()
    spec = importlib.util.spec_from_file_location("config_module", python_file)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return list(module.configs)


def execute_config(config):
    from .train import train
    try:
        return config.run_id, train(config), None
    except Exception:  # noqa: BLE001 - the sweep reports and continues
        return config.run_id, None, traceback.format_exc()


def _worker(gpu, python_file, launch_id, jobs, results):
    if gpu is not None:
        os.environ["CUDA_VISIBLE_DEVICES"] = str(gpu)
    configs = load_configs(python_file)
    while True:
        idx = jobs.get()
        if idx is None:
            return
        configs[idx].launch_id = launch_id
        results.put((idx,) + execute_config(configs[idx]))


def run_sweep(python_file: str, name: str = "default", parallelize: bool = False, gpus: str | None = None) -> list:
    configs = load_configs(python_file)
    launch_id = f"{name}-{datetime.now().strftime('%Y-%m-%d-%H-%M-%S')}"
    print(f"Running sweep {launch_id} with {len(configs)} configs")
    if not parallelize or not configs:
        out = []
        for c in configs:
            c.launch_id = launch_id
            out.append(execute_config(c))
        return out
    if gpus is not None:
        devices = [g for g in gpus.split(",") if g != ""]
    else:
        import torch
        devices = list(range(torch.cuda.device_count())) or [None]
    ctx = mp.get_context("spawn")
    jobs, results = ctx.Queue(), ctx.Queue()
    for i in range(len(configs)):
        jobs.put(i)
    workers = [ctx.Process(target=_worker, args=(g, python_file, launch_id, jobs, results)) for g in devices[:len(configs)]]
    for w in workers:
        jobs.put(None)
        w.start()
    out, failed = [None] * len(configs), 0
    for done in range(1, len(configs) + 1):
        idx, run_id, best, err = results.get()
        out[idx] = (run_id, best, err)
        if err is not None:
            failed += 1
            print(f"config {run_id} failed:\n{err}")
        print(f"Completed: {done} ({done / len(configs):0.1%} -- {failed} failed) | Total: {len(configs)}")
    for w in workers:
        w.join()
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("python_file")
    ap.add_argument("--outdir", default=None)
    ap.add_argument("--name", default="default")
    ap.add_argument("-p", "--parallelize", action="store_true")
    ap.add_argument("--gpus", default=None)
    a = ap.parse_args(argv)
    if a.outdir:
        os.environ.setdefault("ZOOLOGY_CSV", os.path.join(a.outdir, "zoology_results.csv"))
        os.environ.setdefault("ZOOLOGY_LOG_DIR", a.outdir)
    if a.gpus is not None and not a.parallelize:
        os.environ["CUDA_VISIBLE_DEVICES"] = a.gpus
    run_sweep(a.python_file, a.name, a.parallelize, a.gpus)


if __name__ == "__main__":
    main()
