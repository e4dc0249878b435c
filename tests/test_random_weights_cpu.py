"""The counter-based random weights: the package's vectorised generator against the scalar
restatement in tests/plain_qwen2.py (bit-equal), any element alone, and the distribution."""
import numpy as np
import torch

import plain_qwen2 as plain
import replay_util as ru
from dispec_b200.config import load_model_config
from dispec_b200.weights import counter_rng, random_tensors


def test_philox_known_answers():
    zero = np.zeros(1, dtype=np.uint64)
    ones = np.full(1, 0xFFFFFFFF, dtype=np.uint64)
    assert [int(w[0]) for w in counter_rng.philox4x32_10(zero, zero, zero, zero, 0, 0)] == \
        [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert [int(w[0]) for w in counter_rng.philox4x32_10(ones, ones, ones, ones, 0xFFFFFFFF, 0xFFFFFFFF)] == \
        [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert plain._philox4x32_10((0, 0, 0, 0), (0, 0)) == (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)


def test_vectorised_generator_equals_the_scalar_restatement_bit_for_bit():
    for seed, ordinal, start in [(0, 0, 0), (2, 7, 4093), (2 ** 40 + 5, 311, 2 ** 33 + 1), (9, 3, 17)]:
        got = counter_rng.standard_normal(seed, ordinal, 203, start=start)
        want = np.array([plain.counter_normal_element(seed, ordinal, start + i) for i in range(203)], dtype=np.float32)
        assert got.dtype == np.float32 and np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_any_element_alone_and_any_slice_give_the_same_value():
    whole = counter_rng.standard_normal(4, 2, 5000)
    for start, n in [(0, 1), (1, 2), (3, 9), (4997, 3), (1234, 777)]:
        assert np.array_equal(counter_rng.standard_normal(4, 2, n, start=start), whole[start:start + n])
    assert not np.array_equal(counter_rng.standard_normal(4, 3, 100), whole[:100])  # another tensor
    assert not np.array_equal(counter_rng.standard_normal(5, 2, 100), whole[:100])  # another seed


def test_distribution_is_standard_normal():
    z = counter_rng.standard_normal(123, 0, 1_000_000).astype(np.float64)
    assert abs(z.mean()) < 4e-3 and abs(z.std() - 1) < 3e-3
    assert abs((z ** 3).mean()) < 1.5e-2 and abs((z ** 4).mean() - 3) < 4e-2
    for q, p in [(-2.0, 0.02275), (-1.0, 0.158655), (0.0, 0.5), (1.0, 0.841345), (2.5, 0.99379)]:
        assert abs((z < q).mean() - p) < 2e-3
    assert np.abs(np.corrcoef(z[:-1], z[1:])[0, 1]) < 4e-3 and np.abs(np.corrcoef(z[:-2], z[2:])[0, 1]) < 4e-3


def test_model_tensors_follow_the_rule_by_name():
    """A tensor of a random model = mean + std * z(seed, ordinal of its name in sorted order, index),
    rounded once to the storage type; gains have mean 1; an override changes one tensor's std."""
    config = ru.CONFIG_B
    cfg = load_model_config(config)
    tensors = random_tensors(cfg, 1, 0.05, "bfloat16", overrides={"lm_head.weight": 0.5})
    names = list(plain.tensor_shapes(config))
    assert sorted(tensors) == sorted(names)
    probe = [0, 1, 2, 3, 4, 95, 96, 1000]
    for name, std, mean in [("model.layers.1.self_attn.k_proj.weight", 0.05, 0.0),
                            ("model.layers.2.post_attention_layernorm.weight", 0.05, 1.0),
                            ("model.norm.weight", 0.05, 1.0), ("lm_head.weight", 0.5, 0.0),
                            ("model.layers.0.self_attn.q_proj.bias", 0.05, 0.0)]:
        flat = tensors[name].flatten()
        idx = [i for i in probe if i < flat.numel()]
        want = plain.counter_random_tensor(names, name, tensors[name].shape, 1, std, mean, indices=idx)
        assert torch.equal(flat[idx], want.to(torch.bfloat16)), name
    full = random_tensors(cfg, 1, 0.05, "float32")
    name = "model.layers.0.mlp.down_proj.weight"
    assert torch.equal(full[name].flatten()[:64],
                       plain.counter_random_tensor(names, name, full[name].shape, 1, 0.05, indices=range(64)))
