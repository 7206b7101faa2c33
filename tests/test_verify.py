"""Run-time self-checks (hipress_b200/utils/verify.py) on gloo ranks: the replica
checksum and the conservation law ``delivered + mean(kept back) == exact mean`` for
every algorithm that keeps error-feedback state, on both topologies."""
import pytest
import torch

KW = dict(vocab_size=500, hidden=32, layers=2, heads=4, ffn=64, max_pos=32)


def _run(rank, world, alg, topo, break_replica):
    import hipress_b200 as hp
    from hipress_b200.train.harness import build_job
    from hipress_b200.utils.verify import one_step_check, replicas_identical
    cfg = hp.HipressConfig(algorithm=alg, topology=topo, comp_threshold=1000, threshold=1e-4, ratio=0.01)
    job = build_job("bert_base", cfg, batch=2, seq_len=8, dtype=torch.float32, model_kwargs=KW,
                    device=torch.device("cpu"))
    for i in range(2):
        job.step(*job.to_device(*job.host_batch(10 * rank + i)))
    same = replicas_identical(job.model)
    chk = one_step_check(job, *job.to_device(*job.host_batch(77 + rank)))
    if break_replica and rank == 1:
        with torch.no_grad():
            next(job.model.parameters()).view(-1)[0] += 1.0
    broken = replicas_identical(job.model)
    job.optimizer.close()
    return {"same": same, "chk": chk, "after_break": broken}


@pytest.mark.parametrize("alg,topo", [("tbq", "ring"), ("onebit", "ps"), ("dgc", "ps"), ("graddrop", "ring"),
                                      ("dgc", "ring")])
def test_conservation_and_replica_checksum(alg, topo):
    from _mp import spawn
    res = spawn(_run, 2, alg, topo, True)
    for r in res:
        assert r["same"] is True
        assert r["after_break"] is False, "a changed replica must be noticed"
        c = r["chk"]
        assert c["compressed_elems"] > 0 and c["plain_elems"] > 0
        assert c["one_step_rel_err"] < 1e-4, c
        assert c["plain_rel_err"] < 1e-5, c


def test_terngrad_reports_its_quantisation_error():
    from _mp import spawn
    res = spawn(_run, 2, "terngrad", "ring", False)
    for r in res:
        assert r["same"] is True and r["after_break"] is True
        assert 0 < r["chk"]["one_step_rel_err"] < 5.0    # unbiased but noisy: no residual to add back
