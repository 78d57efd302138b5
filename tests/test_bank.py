"""The weight-only recovery map: top-r left singular subspace of all down columns."""

import torch

from cfm_b200.reader.bank import subspace_bank


def test_subspace_bank_matches_a_direct_svd():
    generator = torch.Generator().manual_seed(5)
    experts, hidden, width, rank = 6, 48, 20, 8
    # A spectrum with clear gaps, so the top-r subspace is well defined.
    basis = torch.linalg.qr(torch.randn(hidden, hidden, generator=generator, dtype=torch.float64)).Q
    spectrum = torch.logspace(1, -2, hidden, dtype=torch.float64)
    mixing = torch.randn(hidden, experts * width, generator=generator, dtype=torch.float64)
    columns = basis @ (spectrum[:, None] * mixing)
    down = columns.reshape(hidden, experts, width).permute(1, 0, 2).contiguous()
    decoder, encoder, captured = subspace_bank(down, rank)
    assert decoder.shape == (hidden, rank) and encoder.shape == (experts, rank, width)
    left, singular, _ = torch.linalg.svd(columns, full_matrices=False)
    # Same subspace (signs and rotations inside equal singular values aside) ...
    torch.testing.assert_close(decoder @ decoder.T, left[:, :rank] @ left[:, :rank].T,
                               rtol=0, atol=1e-8)
    # ... ordered by decreasing singular value, orthonormal, encoder = U^T D_e.
    torch.testing.assert_close(decoder.T @ decoder, torch.eye(rank, dtype=torch.float64),
                               rtol=0, atol=1e-10)
    energy = (decoder.T @ columns).square().sum(1)
    assert bool((energy[:-1] >= energy[1:]).all())
    torch.testing.assert_close(encoder[3], decoder.T @ down[3], rtol=0, atol=1e-10)
    expected = float(singular[:rank].square().sum() / singular.square().sum())
    assert abs(captured - expected) < 1e-10
    # What the reader adds for expert e and features p: U B_e p = projection of D_e p.
    features = torch.randn(width, generator=generator, dtype=torch.float64)
    projector = left[:, :rank] @ left[:, :rank].T
    torch.testing.assert_close(decoder @ (encoder[2] @ features), projector @ (down[2] @ features),
                               rtol=0, atol=1e-8)
