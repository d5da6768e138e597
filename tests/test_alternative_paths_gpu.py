"""The library keeps three environment switches that select an alternative kernel for the
same result (used for comparisons when a kernel is tuned):
  FRNNT_CONTRACTION=tf32 | simt   simple lattices on the 3xTF32 engine / on the FMA pipe
                                  instead of the fp16-pair engine,
  FRNNT_MI=row_per_thread         the lattice backward with one row per thread for all sizes,
  FRNNT_PAIR_TILE=128             128 x 128 tiles for every fp16-pair product.
Each alternative must pass the same checks as the default, so that none of them rots."""
import pytest
import torch

from tests import test_joiner_fused_gpu, test_mi_gpu, test_pairs_gpu, test_rnnt_loss_gpu

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["tf32", "simt"])
def test_simple_lattices_on_the_other_engines(monkeypatch, mode):
    monkeypatch.setenv("FRNNT_CONTRACTION", mode)
    test_rnnt_loss_gpu.test_simple_variants()
    for rnnt_type in ("regular", "modified", "constrained"):
        test_rnnt_loss_gpu.test_mini_pipeline_stagewise(rnnt_type)


def test_lattice_backward_with_one_row_per_thread(monkeypatch):
    monkeypatch.setenv("FRNNT_MI", "row_per_thread")
    for modified in (False, True):
        test_mi_gpu.test_mi_random_vs_oracle(torch.float32, modified)
    test_rnnt_loss_gpu.test_mini_pipeline_stagewise("regular")


def test_pair_products_on_small_tiles(monkeypatch):
    monkeypatch.setenv("FRNNT_PAIR_TILE", "128")
    for shape in test_pairs_gpu.NT_SHAPES[2:6]:
        test_pairs_gpu.test_pair_matmul_nt(*shape, True)
    for shape in test_pairs_gpu.TN_SHAPES[1:]:
        test_pairs_gpu.test_pair_matmul_tn(*shape)
    test_joiner_fused_gpu.test_fused_lattices_and_gradients_match_float64((2, 33, 12, 5, 512, 500), "regular")
