"""GPU: the random-weights mode gives the same tensors on the device as in a
folder, bit for bit, in every precision policy; so a model made with
``Session.random`` has a twin that the plain implementation can read."""

import pytest
import torch

from tiny_configs import TINY_B, TINY_D

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("storage", ["float32", "bfloat16"])
@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_device_and_folder_modes_hold_the_same_values(tmp_path, storage, compute):
    from llmoxide_b200 import read_config, write_model_folder
    from llmoxide_b200.weights import load_checkpoint, random_tensors_on_device

    for raw, seed in ((TINY_B, 5), (TINY_D, 6)):
        cfg = read_config(dict(raw, torch_dtype=storage))
        spec = cfg.to_spec()
        folder = write_model_folder(tmp_path / f"m{seed}", cfg, seed)
        loaded = load_checkpoint(folder, spec, compute, "cuda")
        made = random_tensors_on_device(spec, seed, compute, "cuda")
        assert set(loaded) == set(made)
        for name in loaded:
            assert loaded[name].dtype == made[name].dtype, name
            assert torch.equal(loaded[name], made[name]), name
        # another seed gives other values; a gain is around one, a matrix around zero
        other = random_tensors_on_device(spec, seed + 1, compute, "cuda")
        assert not torch.equal(other["model.norm.weight"], made["model.norm.weight"])
        assert abs(float(made["model.norm.weight"].float().mean()) - 1.0) < 0.02
        emb = made["model.embed_tokens.weight"].float()
        assert abs(float(emb.mean())) < 2e-3 and abs(float(emb.std()) - 0.02) < 2e-3


def test_a_tensor_larger_than_one_host_chunk():
    """The host makes large tensors in pieces on several threads; the pieces join without a seam."""
    from llmoxide_b200 import kernels
    from llmoxide_b200.config.spec import TensorSpec
    from llmoxide_b200.weights import random_init as ri

    t = TensorSpec("model.layers.0.mlp.down_proj.weight", (3 * (1 << 22) // 1024 + 7, 1024))
    host = ri.host_tensor(t, 11, torch.bfloat16)
    dev = torch.empty(t.shape, dtype=torch.bfloat16, device="cuda")
    q = torch.from_numpy(ri.quantiles()).cuda()
    kernels.fill_normal(dev, ri._stream_seed(11, t.name), q, 0.0, ri.MATRIX_STD, torch.bfloat16)
    assert torch.equal(dev.cpu(), host)
    x = host.float()
    assert abs(float(x.std()) - 0.02) < 1e-4 and float(x.abs().max()) < 0.02 * 4.6
    # the fourth moment of a normal: 3 sigma^4 (the cut at 4.5 sigma and the straight pieces move it little)
    assert abs(float((x ** 4).mean()) / 0.02 ** 4 - 3.0) < 0.05
