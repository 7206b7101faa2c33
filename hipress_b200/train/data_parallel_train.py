"""Job launcher with the flags of the reference's MXNet launcher
``data_parallel_train.py`` (README.md:45,51,160-169 of mark14wu/hipress):

    python -m hipress_b200.train.data_parallel_train --numprocess 8 \
        --servers localhost:8 --model vgg19 --topo Ring --comp-alg tbq --comp-threshold 262144

The reference starts one process per host over ssh / mpirun / horovodrun.  Here a
host list that names only this machine starts ``--numprocess`` local ranks (one
per GPU) with ``torch.distributed.run``.  A list with other machines
(``node1:8,node2:8``; the same slot count on each) starts one
``torch.distributed.run`` per machine, the remote ones over ssh (``--ssh-port``,
22222 in the reference's setup, README.md:29-39), with the first host as the
rendezvous address; ``--interface`` selects the network interface of NCCL and
gloo, as in the reference.  ``--horovodrun`` is accepted for command-line
compatibility and has no effect.  Flags the launcher does not know
(``--train-dir``, ``--checkpoint-dir``, ``--elastic`` ...) are handed to the
training script.
"""
from __future__ import annotations

import argparse
import os
import shlex
import socket
import subprocess
import sys


def parse_servers(text: str):
    out = []
    for item in text.split(","):
        host, _, slots = item.strip().partition(":")
        out.append((host, int(slots or 1)))
    return out


def _train_args(a) -> list[str]:
    args = ["-m", "hipress_b200.train.pytorch_imagenet",
            "--model", a.model, "--topo", a.topo, "--comp-alg", a.comp_alg,
            "--comp-threshold", str(a.comp_threshold), "--num-iterations", str(a.num_iterations),
            "--epochs", str(a.epochs)]
    if a.batch_size:
        args += ["--batch-size", str(a.batch_size)]
    if a.comprplan:
        args += ["--comprplan", a.comprplan]
    return args + list(getattr(a, "extra", []))   # anything else goes to the training script


def _is_local(host: str) -> bool:
    return host in {"localhost", "127.0.0.1", socket.gethostname()}


def build_command(a) -> list[str]:
    """The single-machine command (every host of ``--servers`` is this machine)."""
    servers = parse_servers(a.servers) if a.servers else [("localhost", a.numprocess)]
    foreign = [h for h, _ in servers if not _is_local(h)]
    if foreign:
        raise SystemExit(f"hosts {foreign} are not this machine: use build_commands()")
    slots = sum(s for _, s in servers)
    if slots < a.numprocess:
        raise SystemExit(f"--servers offers {slots} slots for --numprocess {a.numprocess}")
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
            f"--nproc-per-node={a.numprocess}", "--master-addr", "127.0.0.1",
            "--master-port", str(a.port), *_train_args(a)]


def build_commands(a) -> list[tuple[str, list[str]]]:
    """(host, argv) per machine.  One entry for a single-machine job; otherwise one
    ``torch.distributed.run`` per machine, wrapped in ssh for the remote ones."""
    servers = parse_servers(a.servers) if a.servers else [("localhost", a.numprocess)]
    if all(_is_local(h) for h, _ in servers):
        return [("localhost", build_command(a))]
    hosts = list(dict.fromkeys(h for h, _ in servers))
    if len(hosts) != len(servers):
        raise SystemExit("--servers names a machine twice")
    per = {s for _, s in servers}
    if len(per) != 1:
        raise SystemExit("every machine must offer the same number of slots")
    per = per.pop()
    if per * len(servers) != a.numprocess:
        raise SystemExit(f"--servers offers {per * len(servers)} slots for --numprocess {a.numprocess}")
    master = "127.0.0.1" if _is_local(hosts[0]) and len(hosts) == 1 else hosts[0]
    env = []
    if a.interface:
        env = [f"NCCL_SOCKET_IFNAME={a.interface}", f"GLOO_SOCKET_IFNAME={a.interface}"]
    out = []
    for k, host in enumerate(hosts):
        run = ["python", "-m", "torch.distributed.run", f"--nnodes={len(hosts)}", f"--node-rank={k}",
               f"--nproc-per-node={per}", "--master-addr", master, "--master-port", str(a.port),
               *_train_args(a)]
        if _is_local(host):
            out.append((host, ["env", *env, sys.executable, *run[1:]]))
        else:
            remote = " ".join(["cd", shlex.quote(os.getcwd()), "&&", "env", *env, *map(shlex.quote, run)])
            out.append((host, ["ssh", "-p", str(a.ssh_port), "-o", "StrictHostKeyChecking=no", host, remote]))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description="hipress_b200 data-parallel launcher")
    ap.add_argument("--numprocess", type=int, default=1)
    ap.add_argument("--servers", default=None, help="host:slots,...")
    ap.add_argument("--ssh-port", type=int, default=22222, help="ssh port of the other machines")
    ap.add_argument("--model", default="vgg19")
    ap.add_argument("--topo", default="Ring", choices=["PS", "Ring", "ps", "ring", "RING"])
    ap.add_argument("--comp-alg", default="tbq")
    ap.add_argument("--comp-threshold", type=int, default=262144)
    ap.add_argument("--comprplan", default=None)
    ap.add_argument("--horovodrun", action="store_true", help="accepted, no effect")
    ap.add_argument("--interface", default=None, help="network interface for NCCL / gloo sockets")
    ap.add_argument("--batch-size", type=int, default=None)
    ap.add_argument("--num-iterations", type=int, default=20)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--port", type=int, default=29500)
    ap.add_argument("--dry-run", action="store_true", help="print the command and exit")
    a, a.extra = ap.parse_known_args(argv)
    cmds = build_commands(a)
    if a.dry_run:
        for _, cmd in cmds:
            print(" ".join(cmd))
        return 0
    os.makedirs("trainResult", exist_ok=True)
    procs = [subprocess.Popen(cmd) for _, cmd in cmds]
    return max(p.wait() for p in procs)


if __name__ == "__main__":
    sys.exit(main())
