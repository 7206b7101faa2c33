"""Command line of the planner, same flags and file formats as the reference's
``python SeCoPa.py --input --output --topology PS|RING --nnodes N``
(src/SeCoPa/SeCoPa.py:116-137), plus ``--profile`` to use coefficients measured on
this machine instead of the reference's."""
import argparse

from .planner import CostProfile, Planner, format_plan, read_gradient_list, reference_profile


def main(argv=None):
    ap = argparse.ArgumentParser(description="SeCoPa: selective compression and partitioning",
                                 formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("--input", default="input.txt", help="rows of name,size")
    ap.add_argument("--model", default=None,
                    help="take the gradient list from a model of the zoo (vgg19, resnet50, bert_large, "
                         "...) instead of --input")
    ap.add_argument("--output", default="SeCoPaPlan.txt", help="rows of name,size,y|n,K")
    ap.add_argument("--topology", default="PS", choices=["PS", "RING"])
    ap.add_argument("--nnodes", type=int, default=16, help="cluster size")
    ap.add_argument("--profile", default="reference",
                    help="'reference' or a JSON file written by hipress_b200.secopa.profiler")
    ap.add_argument("--bucketed", action="store_true",
                    help="decide jointly for a bucketed runtime (measured profiles only)")
    ap.add_argument("--bucket-mb", type=int, default=256, help="--bucketed: gradient MB per fused launch")
    a = ap.parse_args(argv)
    if a.profile == "reference":
        prof = reference_profile(a.nnodes)
    else:
        with open(a.profile) as f:
            prof = CostProfile.from_json(f.read())
        if prof.nodes != a.nnodes:
            raise SystemExit(f"profile was measured for {prof.nodes} nodes, not {a.nnodes}")
    if a.model:
        from ..models import get_model
        from .planner import gradient_list_of
        m = get_model(a.model)
        named = m.gluon_named_parameters() if hasattr(m, "gluon_named_parameters") else m.named_parameters()
        grads = gradient_list_of((n, p) for n, p in named if p.requires_grad)
    else:
        grads = read_gradient_list(a.input)
    if a.bucketed:
        rows = Planner(prof).plan_bucketed(grads, a.topology, a.bucket_mb << 20)
    else:
        rows = Planner(prof).plan(grads, a.topology)
    with open(a.output, "w") as f:
        f.write(format_plan(rows))


if __name__ == "__main__":
    main()
