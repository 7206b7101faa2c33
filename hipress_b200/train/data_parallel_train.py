"""Job launcher with the flags of the reference's MXNet launcher
``data_parallel_train.py`` (README.md:45,51,160-169 of mark14wu/hipress):

    python -m hipress_b200.train.data_parallel_train --numprocess 8 \
        --servers localhost:8 --model vgg19 --topo Ring --comp-alg tbq --comp-threshold 262144

The reference starts one process per host over ssh / mpirun / horovodrun; this
framework targets one NVSwitch box, so the launcher starts ``--numprocess`` local
ranks (one per GPU) with ``torch.distributed.run`` and rejects host lists that
name another machine.  ``--interface`` and ``--horovodrun`` are accepted for
command-line compatibility and have no effect on a single box.
"""
from __future__ import annotations

import argparse
import os
import socket
import subprocess
import sys


def parse_servers(text: str):
    out = []
    for item in text.split(","):
        host, _, slots = item.strip().partition(":")
        out.append((host, int(slots or 1)))
    return out


def build_command(a) -> list[str]:
    local = {"localhost", "127.0.0.1", socket.gethostname()}
    servers = parse_servers(a.servers) if a.servers else [("localhost", a.numprocess)]
    foreign = [h for h, _ in servers if h not in local]
    if foreign:
        raise SystemExit(f"hosts {foreign} are not this machine: hipress_b200 runs on one NVSwitch box")
    slots = sum(s for _, s in servers)
    if slots < a.numprocess:
        raise SystemExit(f"--servers offers {slots} slots for --numprocess {a.numprocess}")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={a.numprocess}", "--master-addr", "127.0.0.1",
           "--master-port", str(a.port), "-m", "hipress_b200.train.pytorch_imagenet",
           "--model", a.model, "--topo", a.topo, "--comp-alg", a.comp_alg,
           "--comp-threshold", str(a.comp_threshold), "--num-iterations", str(a.num_iterations),
           "--epochs", str(a.epochs)]
    if a.batch_size:
        cmd += ["--batch-size", str(a.batch_size)]
    if a.comprplan:
        cmd += ["--comprplan", a.comprplan]
    return cmd


def main(argv=None):
    ap = argparse.ArgumentParser(description="hipress_b200 data-parallel launcher")
    ap.add_argument("--numprocess", type=int, default=1)
    ap.add_argument("--servers", default=None, help="host:slots,... (this machine only)")
    ap.add_argument("--model", default="vgg19")
    ap.add_argument("--topo", default="Ring", choices=["PS", "Ring", "ps", "ring", "RING"])
    ap.add_argument("--comp-alg", default="tbq")
    ap.add_argument("--comp-threshold", type=int, default=262144)
    ap.add_argument("--comprplan", default=None)
    ap.add_argument("--horovodrun", action="store_true", help="accepted, no effect")
    ap.add_argument("--interface", default=None, help="accepted, no effect")
    ap.add_argument("--batch-size", type=int, default=None)
    ap.add_argument("--num-iterations", type=int, default=20)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--port", type=int, default=29500)
    ap.add_argument("--dry-run", action="store_true", help="print the command and exit")
    a = ap.parse_args(argv)
    cmd = build_command(a)
    if a.dry_run:
        print(" ".join(cmd))
        return 0
    os.makedirs("trainResult", exist_ok=True)
    return subprocess.call(cmd)


if __name__ == "__main__":
    sys.exit(main())
