"""Host-side pieces of bench.py that need no GPU: the defaults the contract asks for, the synthetic routing of the
prefill workload, the byte accounting of the FP8 roofline and the CPU arm's independence of its thread count."""
import sys

import numpy as np

import bench


def test_defaults_are_one_gpu_and_a_few_steps(monkeypatch):
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = bench.parse_args()
    assert args.gpus == 1 and args.impl == "ours"
    assert args.warmup >= 3 and 1 <= args.steps <= 100


def test_zipf_routing_draws_distinct_experts_and_normalised_weights():
    ids, w = bench.zipf_routing(np.random.default_rng(3), 512, 384, 6)
    assert ids.shape == (512, 6) and ids.dtype == np.int32 and w.shape == (512, 6) and w.dtype == np.float32
    assert ids.min() >= 0 and ids.max() < 384
    assert all(len(set(row)) == 6 for row in ids.tolist())            # six DISTINCT experts per token
    np.testing.assert_allclose(w.sum(1), 1.0, rtol=1e-6)
    # skewed popularity: the busiest expert gets far more than the mean share of 6/384 of the tokens
    counts = np.bincount(ids.reshape(-1), minlength=384)
    assert counts.max() > 8 * counts.mean()
    ids2, w2 = bench.zipf_routing(np.random.default_rng(3), 512, 384, 6)
    assert (ids == ids2).all() and (w == w2).all()                     # seeded: the same stream again


def test_fp8_algorithmic_bytes_count_weights_scales_activations_and_output():
    n, k, b = 12288, 4096, 1
    got = bench.fp8_alg_bytes(n, k, b)
    weights, scales = n * k, (n // 128) * (k // 128) * 4
    assert got >= weights + scales
    assert got - weights - scales <= b * (k * 2 + k // 128 * 4 + k + n * 2) + 64   # activations in, their codes/scales, bf16 out
    assert bench.fp8_alg_bytes(n, k, 32) > got


def test_cpu_arm_gives_the_same_layer_output_for_any_thread_count(monkeypatch):
    # a small layer: the arm's arithmetic per expert does not depend on how the experts are spread over threads
    monkeypatch.setattr(bench, "HIDDEN", 256)
    monkeypatch.setattr(bench, "INTER", 128)
    monkeypatch.setattr(bench, "EXPERTS", 16)
    monkeypatch.setattr(bench, "TOPK", 4)
    for kind in ("affine2", "fp4"):
        x, w, experts = bench.cpu_layer_inputs(kind, seed=5)
        assert x.shape == (256,) and len(experts) == 4 and abs(float(np.sum(w)) - 1.0) < 1e-5
        one = bench.cpu_layer_pass(kind, x, w, experts, threads=1)
        many = bench.cpu_layer_pass(kind, x, w, experts, threads=4)
        assert one.shape == (256,) and np.isfinite(one).all() and np.abs(one).max() > 0
        assert (one == many).all()
