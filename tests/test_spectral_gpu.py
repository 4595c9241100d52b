"""K4 spectral key codec on the GPU against the reference-made vectors and the oracle: containers are
the reference's, codes differ only at rounding ties of the float32 encode, dequant agrees to 1e-5."""

import numpy as np
import pytest
import torch

from oracle import bmx_oracle as O
from tests.helpers import golden

pytestmark = pytest.mark.gpu


def test_spectral_append_and_dequant_vs_reference_vectors():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K

    dev, c = torch.device("cuda:0"), golden("spectral")
    bits = torch.from_numpy(c["bits"]).to(torch.int32)
    # two heads: head 0 carries the reference's pack and data, head 1 a second seeded pack
    g = torch.Generator().manual_seed(9)
    Q2, _ = torch.linalg.qr(torch.randn(128, 128, generator=g))
    perm = torch.randperm(128, generator=g)
    enc = torch.stack([torch.from_numpy(c["E"]), Q2]).contiguous()
    dec = torch.stack([torch.from_numpy(c["dec8"]), Q2]).contiguous()
    bits2 = torch.stack([bits, bits[perm]])
    pack = K.SpectralPackDev(enc, dec, bits2, page=128, group=64, device=dev)
    M0 = torch.from_numpy(c["M"])
    M1 = torch.randn(128, 128, generator=g) * 0.5
    k_pre = torch.stack([M0, M1])[None].contiguous()  # (1, 2, 128, 128) float32 source
    pool = pack.new_pool(4)
    slots = torch.tensor([2], dtype=torch.int32, device=dev)
    K.spectral_append(pack, pool, k_pre.to(dev), slots, 1)
    out = K.spectral_dequant_pages(pack, pool, slots)
    codes, scales, kd = out["codes"][0].cpu(), out["scales"][0].cpu(), out["k"][0].cpu().numpy()
    # ---- head 0 against the reference's packed dict ----
    d0 = {a: t.cpu().numpy() for a, t in K.spectral_tier_dict(pack, out["codes"][0, 0], out["scales"][0, 0], 0).items()}
    ref_keys = sorted(k[2:] for k in c.files if k.startswith("p_"))
    assert sorted(d0) == ref_keys, "same tiers and containers as the reference's packed dict"
    for name in ref_keys:
        ref = c["p_" + name]
        assert d0[name].shape == ref.shape and d0[name].dtype == ref.dtype, name
        if name.endswith("_codes"):
            assert (d0[name] != ref).mean() < 5e-3, name          # bytes differ only at rounding ties
        else:
            np.testing.assert_allclose(d0[name], ref, rtol=2e-4)  # refined float32 steps
    # dequant of OUR stored fields through the oracle's decode: same float32 sums in another order
    ref_deq = O.spectral_dequant_packed(d0, c["dec8"], c["bits"], 64)
    assert np.abs(kd[:, :128] - ref_deq).max() <= 1e-5 * np.abs(ref_deq).max()
    # and close to the reference's own reconstruction (its codes differ at a few ties)
    assert np.abs(kd[:, :128] - c["deq"]).max() <= 0.05 * np.abs(c["deq"]).max()
    # ---- head 1 against the oracle end to end ----
    p1 = O.spectral_quantize_packed(M1.numpy(), Q2.numpy(), bits2[1].numpy(), 64)
    d1 = {a: t.cpu().numpy() for a, t in K.spectral_tier_dict(pack, out["codes"][0, 1], out["scales"][0, 1], 1).items()}
    for name in p1:
        if name.endswith("_codes"):
            assert (d1[name] != p1[name]).mean() < 5e-3, name
        else:
            np.testing.assert_allclose(d1[name], p1[name], rtol=2e-4)
    ref1 = O.spectral_dequant_packed(d1, Q2.numpy(), bits2[1].numpy(), 64)
    assert np.abs(kd[:, 128:] - ref1).max() <= 1e-5 * np.abs(ref1).max()
    # code ranges per tier, and directions without bits decode to nothing
    for b in (2, 3, 4, 5, 6, 8):
        sel = bits2[0] == b
        if sel.any():
            qmax = 2 ** (b - 1) - 1
            assert codes[0][sel].min() >= -qmax - 1 and codes[0][sel].max() <= qmax
    assert (codes[0][bits2[0] == 0] == 0).all() and (scales[0][bits2[0] == 0] == 0).all()
