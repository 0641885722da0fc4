"""Generated K x K Hadamard matrices equal the ones the reference stores (golden: had12/20/28
in full, every other order by digest)."""
import hashlib

import numpy as np
import pytest
import torch

from gptq_plus_mp_quant_b200.utils import hadamard_utils as hu


def _sha(mat) -> str:
    return hashlib.sha256(np.ascontiguousarray(np.asarray(mat, dtype=np.int8)).tobytes()).hexdigest()[:16]


def test_table_orders_match_reference(golden):
    g = golden("hadamard.npz")
    assert tuple(int(k) for k in g["table_keys"]) == hu.TABLE_ORDERS


@pytest.mark.parametrize("K", [12, 20, 28])
def test_small_orders_bit_equal(golden, K):
    g = golden("hadamard.npz")
    assert torch.equal(hu.hadamard_of_order(K), torch.from_numpy(g[f"had{K}"]).float())


def test_generated_orders_match_digests(golden):
    g = golden("hadamard.npz")
    for K in hu.TABLE_ORDERS:                        # all thirty orders: generated or unpacked from the table
        H = hu.hadamard_of_order(K)
        assert _sha(H.numpy()) == str(g[f"had_sha.{K}"]), f"order {K} differs from the reference table"
        assert torch.equal(H @ H.T, K * torch.eye(K))
    with pytest.raises(ValueError):
        hu.hadamard_of_order(24)


@pytest.mark.parametrize("n,K", [(4096, 1), (12288, 12), (28672, 28), (5120, 20), (128, 1), (9216, 36), (11008, 172)])
def test_get_hadK_picks_smallest_factor(n, K):
    hadK, k = hu.get_hadK(n)
    assert k == K
    assert (hadK is None) == (K == 1)


def test_random_orthogonal_matrix():
    """hadamard_utils.py:56-73: orthogonal in fp64, reproducible from the generator, sign convention of R's diagonal."""
    g = torch.Generator().manual_seed(3)
    q = hu.random_orthogonal_matrix(48, "cpu", generator=g)
    assert q.dtype == torch.float64 and q.shape == (48, 48)
    assert torch.allclose(q @ q.T, torch.eye(48, dtype=torch.float64), atol=1e-12)
    gauss = torch.randn(48, 48, dtype=torch.float64, generator=torch.Generator().manual_seed(3))
    assert bool((torch.diagonal(q.T @ gauss) > 0).all())            # R = Q^T A has a positive diagonal
    assert torch.equal(q, hu.random_orthogonal_matrix(48, "cpu", generator=torch.Generator().manual_seed(3)))
