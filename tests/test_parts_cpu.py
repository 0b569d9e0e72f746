"""The tests of tests/test_parts_gpu.py once more, on the CPU with torch stand-ins for the
kernels (tests/cpu_ops.py): each part alone, a block against the plain layer, and the generality of the
assembly (a layer run twice, a shared cache, a windowed group that gives pages back, other position
encodings, the toy mixer with state, the toy routed feed-forward, the toy position encoding).  What they check here is the Python
above the kernels; the kernels themselves are checked on the GPU."""

import functools

import pytest
import torch

from dli_b200.engine import random_model
from tests import cpu_ops
from tests import test_parts_gpu as g
from tests.tiny_configs import TINY_A, TINY_B, TINY_C

F32 = torch.float32
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(autouse=True)
def on_the_cpu(monkeypatch):
    monkeypatch.setattr(g, "DEV", torch.device("cpu"))
    monkeypatch.setattr(g, "random_model", functools.partial(random_model, device="cpu"))
    with cpu_ops.patched():
        yield


@pytest.mark.parametrize("dtype", DTYPES, ids=["float32", "bfloat16"])
def test_norm_feed_forward_embedding_and_head(dtype):
    g.test_norm_part(dtype)
    g.test_feed_forward_part(dtype)
    g.test_embedding_and_head_parts(dtype, True)
    g.test_embedding_and_head_parts(dtype, False)


@pytest.mark.parametrize("dtype", DTYPES, ids=["float32", "bfloat16"])
@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C], ids=["a", "b", "c"])
def test_frequencies_and_block(cfg, dtype):
    g.test_rotary_part_frequencies(cfg)
    g.test_block_of_parts_equals_plain_layer(dtype, cfg)


@pytest.mark.parametrize("dtype", DTYPES, ids=["float32", "bfloat16"])
@pytest.mark.parametrize("rotary_dim", [0, 16])
def test_other_position_encodings(rotary_dim, dtype):
    g.test_other_position_encodings(dtype, rotary_dim)


@pytest.mark.parametrize("dtype", DTYPES, ids=["float32", "bfloat16"])
def test_run_order_and_window(dtype):
    g.test_run_order_names_a_layer_twice_and_shares_a_cache(dtype)
    g.test_windowed_layer_has_pages_of_its_own_and_gives_them_back(dtype)
    g.test_unknown_part_kind_is_named()


@pytest.fixture
def toy_architecture():
    """As the fixture of the same name in tests/test_parts_gpu.py."""
    g.register_part("mixer", "toy_running_mean")(g.RunningMean)
    g.register_architecture(g.Architecture("ToyStateLM", g.LlamaConfig.from_hf_dict, lambda cfg: g.toy_spec(cfg.to_hf_dict())))
    yield {**TINY_B, "architectures": ["ToyStateLM"]}
    g.unregister_architecture("ToyStateLM")
    g.unregister_part("mixer", "toy_running_mean")


def test_toy_parts(toy_architecture):
    g.test_toy_mixer_with_state_is_registered_built_and_stepped(toy_architecture)
    g.test_toy_routed_feed_forward_is_registered_and_stepped()


@pytest.mark.parametrize("dtype", DTYPES, ids=["float32", "bfloat16"])
def test_toy_position_encoding(dtype):
    g.test_toy_position_encoding_with_a_table_is_registered_and_stepped(dtype)


def test_toy_layer_with_pages_and_state_and_toy_mixer_with_a_launch_key():
    g.test_a_layer_may_keep_pages_and_a_state_slot()
    g.test_a_toy_mixer_with_its_own_launch_key_decodes_through_graphs()
