"""The memory plan is made from the model's own parts (the tensors they declare, what their mixers keep per token),
so it works for an architecture that is registered from outside the package. Needs no GPU."""

import json

import pytest
import torch

from test_toy_architecture_gpu import LATENT, ROUTED, TOY, latent_state, register_latent_toy, register_routed_toy, register_toy, routed_state, toy_state


def _bytes(state, itemsize):
    return sum(t.numel() * (itemsize if t.dim() == 2 else 4) for t in state.values())


@pytest.mark.parametrize("dtype,itemsize", [("float32", 4), ("bfloat16", 2)])
def test_plan_memory_for_architectures_registered_by_a_test(dtype, itemsize):
    from stride_b200.config import PlanError, config_from_dict, plan_memory
    register_toy(), register_routed_toy(), register_latent_toy()
    gib = 1 << 30
    # routed toy: attention in every layer, keys and values of num_kv_heads x head_dim
    plan = plan_memory(config_from_dict(ROUTED), dtype, memory_bytes=gib, block_size=8, activation_fraction=0.25)
    assert plan.weight_bytes == _bytes(routed_state(1), itemsize)
    assert plan.kv_bytes_per_token == ROUTED["layers"] * 2 * ROUTED["num_kv_heads"] * ROUTED["head_dim"] * itemsize
    left = gib - plan.weight_bytes
    assert plan.activation_reserve_bytes == int(left * 0.25)
    assert plan.num_blocks == (left - int(left * 0.25)) // (plan.kv_bytes_per_token * 8)
    # latent toy: one vector per token and layer, and a head with a bias
    plan = plan_memory(config_from_dict(LATENT), dtype, memory_bytes=gib, block_size=8)
    assert plan.weight_bytes == _bytes(latent_state(1), itemsize)
    assert plan.kv_bytes_per_token == LATENT["layers"] * LATENT["latent"] * itemsize
    # running-mean toy: layer 0 runs twice with a cache slot each, layer 1 keeps no pages but a float32 state per request
    plan = plan_memory(config_from_dict(TOY), dtype, memory_bytes=gib, block_size=8, max_requests=10)
    assert plan.weight_bytes == _bytes(toy_state(1), itemsize) + 10 * TOY["hidden_size"] * 4
    assert plan.kv_bytes_per_token == 2 * 2 * TOY["num_kv_heads"] * TOY["head_dim"] * itemsize
    with pytest.raises(PlanError, match="the weights need"):
        plan_memory(config_from_dict(ROUTED), dtype, memory_bytes=1000)


def test_the_plan_command_for_an_architecture_registered_by_a_test(tmp_path, capsys):
    from stride_b200 import cli
    register_routed_toy()
    path = tmp_path / "config.json"
    path.write_text(json.dumps(ROUTED))
    assert cli.main(["plan", "--config", str(path), "--dtype", "float32", "--memory-gib", "0.5", "--block-size", "8", "--context", "96"]) == 0
    out = capsys.readouterr().out
    assert "bytes a token" in out and "requests of 96" in out
