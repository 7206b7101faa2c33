"""hipress_b200: compression-aware gradient synchronisation for data-parallel
PyTorch training on one NVSwitch box of B200 GPUs.

Typical use (one process per GPU, launched with ``python -m torch.distributed.run``)::

    import hipress_b200 as hp
    hp.init()
    opt = hp.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.01),
                                  named_parameters=model.named_parameters(),
                                  algorithm="tbq", topology="ring", comp_threshold=262144)
    hp.broadcast_parameters(model.state_dict(), root_rank=0)
    loss.backward(); opt.step(); opt.zero_grad()
"""
from .config import HipressConfig, add_hipress_args, config_from_args  # noqa: F401
from .parallel.comm import (allgather, allgather_object, allreduce, allreduce_, barrier,  # noqa: F401
                            broadcast, broadcast_object, broadcast_optimizer_state,
                            broadcast_parameters, device, init, is_initialized, local_rank,
                            local_size, rank, shutdown, size)
from .parallel.optimizer import DistributedOptimizer  # noqa: F401

# the reference's MXNet front end calls the same wrapper DistributedTrainer
DistributedTrainer = DistributedOptimizer
from .parallel.engine import GradSyncEngine  # noqa: F401
from .ops import (Compressor, algorithm_names, get_algorithm, register_algorithm,  # noqa: F401
                  unregister_algorithm)

__version__ = "0.1.0"
