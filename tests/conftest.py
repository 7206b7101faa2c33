import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "multigpu: needs at least 2 CUDA devices")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        ngpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        ngpu = 0
    for item in items:
        if "multigpu" in item.keywords:
            item.add_marker(pytest.mark.gpu)
            if ngpu < 2:
                item.add_marker(pytest.mark.skip(reason="needs >= 2 GPUs"))
        elif "gpu" in item.keywords and ngpu < 1:
            item.add_marker(pytest.mark.skip(reason="needs a GPU"))


@pytest.fixture(scope="session")
def vgg19_gradient_list(tmp_path_factory):
    """The planner input for VGG-19 (gradient name, element count), generated from
    the model definition with the reference's gradient naming."""
    from hipress_b200.models.vgg import VGG19
    from hipress_b200.secopa import gradient_list_of, write_gradient_list
    import torch
    with torch.device("meta"):
        m = VGG19()
    path = tmp_path_factory.mktemp("secopa") / "vgg19_gradients.txt"
    write_gradient_list(path, gradient_list_of(m.gluon_named_parameters()))
    return path
