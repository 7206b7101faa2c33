"""From DSL source to data-parallel training with a new compression algorithm.

The walk-through of the reference's tutorial (write the algorithm in the DSL,
generate the operators, register them, train with them: README.md:190-277 of
mark14wu/hipress) as one runnable script:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m hipress_b200.compll.examples.train_with_new_algorithm --steps 30

1. ``Int8Encode.pse`` / ``Int8Decode.pse`` next to this file describe 8-bit linear
   quantisation in a dozen lines each.
2. The generator turns them into sm_100a kernels and C++ (rank 0 builds, the others wait).
3. ``hp.register_algorithm`` makes the pair an algorithm of the synchronisation
   runtime: merging, error feedback and the PS owner's re-encode are composed
   around it.
4. ``DistributedOptimizer(algorithm="int8")`` trains a small MLP on synthetic data;
   rank 0 prints one JSON line with the first and last loss.

Runs on CPU ranks (gloo) and on GPUs (NCCL) alike: the binding picks the target
from the tensors' device.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import tempfile
from pathlib import Path

import torch

import hipress_b200 as hp
from hipress_b200.compll import generate_files

HERE = Path(__file__).resolve().parent


def _binding(outdir: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, outdir / name / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return getattr(mod, name)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--topo", default="ring", choices=["ring", "ps"])
    ap.add_argument("--out", default=None, help="directory for the generated operators")
    a = ap.parse_args(argv)

    hp.init()
    dev = hp.device()
    out = Path(a.out or Path(tempfile.gettempdir()) / "hipress_compll_example")
    target = "all" if dev.type == "cuda" else "cpu"
    if hp.rank() == 0:                       # steps 1-2: DSL -> operators
        for name in ("Int8Encode", "Int8Decode"):
            generate_files(HERE / f"{name}.pse", out, build=True, target=target)
    hp.barrier()
    hp.register_algorithm("int8", encode=_binding(out, "Int8Encode"), decode=_binding(out, "Int8Decode"),
                          payload_bytes=lambda n: 4 + n, error_feedback=True, seeded=True)   # step 3

    torch.manual_seed(0)                     # step 4: train
    model = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.Tanh(), torch.nn.Linear(256, 8)).to(dev)
    opt = hp.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9),
                                  model.named_parameters(), algorithm="int8", topology=a.topo,
                                  comp_threshold=1024)
    hp.broadcast_parameters(model.state_dict(), root_rank=0)
    teacher = torch.nn.Linear(64, 8).to(dev)
    gen = torch.Generator(device="cpu").manual_seed(100 + hp.rank())
    losses = []
    for _ in range(a.steps):
        x = torch.randn(128, 64, generator=gen).to(dev)
        with torch.no_grad():
            y = teacher(x)
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(model(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    digest = torch.cat([p.detach().reshape(-1) for p in model.parameters()]).double().sum().item()
    same = len({round(d, 9) for d in hp.allgather_object(digest)}) == 1
    stats = opt.engine.stats()
    if hp.rank() == 0:
        print(json.dumps({"algorithm": "int8", "ranks": hp.size(), "backend": stats["backend"],
                          "compressed_fraction": round(stats["compressed_elems"] / stats["total_elems"], 3),
                          "first_loss": round(losses[0], 5), "last_loss": round(losses[-1], 5),
                          "replicas_identical": same}))
    opt.close()
    hp.shutdown()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
