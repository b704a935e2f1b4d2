import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # GPU tests never run by accident on a machine without a device
    try:
        import torch
        has = torch.cuda.is_available()
    except Exception:
        has = False
    if has:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Tiny random models written once per session into a temporary folder:
    {name: {"float32": dir, "bfloat16": dir}}.  The float32 folder stores the bfloat16 folder's
    values widened, so both engine dtypes and the plain implementation see the same weights."""
    import tiny_configs
    from kestrel_llm_b200.config import Qwen3Config
    from kestrel_llm_b200.weights import write_random_model
    from kestrel_llm_b200.weights.safetensors_io import ModelFolder, write_safetensors
    import shutil
    import torch
    out = {}
    for name, (raw, seed) in tiny_configs.CONFIGS.items():
        cfg = Qwen3Config.from_dict(raw)
        base = tmp_path_factory.mktemp(f"model_{name}")
        d16 = str(base / "bf16")
        d32 = str(base / "f32")
        write_random_model(cfg, seed, d16, "bfloat16")
        os.makedirs(d32)
        shutil.copy(os.path.join(d16, "config.json"), os.path.join(d32, "config.json"))
        mf = ModelFolder(d16)
        write_safetensors(os.path.join(d32, "model.safetensors"),
                          ((n, mf.tensor(n).to(torch.float32)) for n in mf.names()))
        mf.close()
        out[name] = {"bfloat16": d16, "float32": d32}
    return out
