"""Layer steps at the FULL shapes of the benchmark configurations vs the oracle pipeline on the
same seeded inputs (masks and cache indices bit-exact, outputs within 1e-5 fp32 / 2e-2 16-bit).
Few steps each, so that the scalar CPU oracle stays within a minute:
  C1  Llama-3.2-1B layer, fp32, one row, all 128 steps of the configuration
  C3  Mistral-7B layer, bf16, 8 rows (H = 4096: the six-neuron tile configuration of k_mlp_bn)
  C5  the same layer with 64 rows on one GPU: the tcgen05 row-block step on the packed cache with the
      device-side K
(C2, Llama-3.2-3B shape, one row: tests/test_gpu_stack.py::test_c2_full_shape_16_steps.)"""
import numpy as np
import pytest

from test_gpu_layer import _run

pytestmark = pytest.mark.gpu


def test_c1_all_128_steps():
    from sparse_transformers_b200.synth import WORKLOADS

    w = WORKLOADS["C1"]
    ks = _run(w, steps=w.steps)
    assert len(ks) == 128 and 0.15 * w.I < np.mean(ks[4:]) < 0.25 * w.I


def test_c3_full_shape_eight_rows():
    from sparse_transformers_b200.synth import WORKLOADS

    w = WORKLOADS["C3"].scaled(layers=1)
    ks = _run(w, steps=3)
    assert 0.3 * w.I < np.mean(ks) < 0.7 * w.I  # union of 8 masks that share 70 % of their variance


def test_c5_full_shape_sixty_four_rows_one_gpu():
    from sparse_transformers_b200.synth import WORKLOADS

    w = WORKLOADS["C5"].scaled(layers=1)
    ks = _run(w, steps=2)
    assert 0.4 * w.I < np.mean(ks) < 0.9 * w.I
