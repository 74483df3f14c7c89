"""Scale-factor and packed-code layout of the oracle."""
import hashlib
import json
import os

import numpy as np
import torch

from oracle import oracle as O


def test_sf_offsets_match_memory_order_enumeration(golden_dir):
    gold = json.load(open(os.path.join(golden_dir, "sf_layout.json")))
    for key, ent in gold.items():
        rows, k_eff = map(int, key.split("x"))
        ncols = k_eff // 16
        t = np.array([[O.sf_offset(r, c, ncols) for c in range(ncols)] for r in range(rows)], dtype="<i8")
        assert hashlib.sha256(t.tobytes()).hexdigest() == ent["sha256"], key
        for r, c, off in ent["spots"]:
            assert t[r, c] == off
        # a bijection onto a prefix-dense set: no two scales share a byte
        assert len(np.unique(t)) == t.size


def test_sf_sizes_follow_the_reference_formula():
    assert O.sf_bytes_reference(512, 4224) == 168960          # (512/128+1)*128*264
    assert O.sf_bytes_span(512, 4224) == 4 * 66 * 512         # 135168 valid bytes
    assert O.sf_alloc_bytes(128, 4224) >= O.sf_bytes_span(128, 4224)
    assert O.sf_bytes_span(1, 14464) == 226 * 512


def test_worked_layout_example_kq4096_ke128():
    """One packed row is 2112 bytes: 1984 bytes of plain groups, then 8 x (8 B main, 8 B residual);
    264 scale columns, column 248 = main of critical group 0, 249 = its residual."""
    kq, ke = 4096, 128
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(3, kq, generator=g) * 4).to(torch.bfloat16)
    idx = torch.randperm(kq, generator=g).to(torch.int16).numpy()
    q, sf = O.quantize_x(x, idx, ke, fill=0xEE)
    assert q.shape == (3, 2112)
    xg = x[:, torch.from_numpy(idx.astype(np.int64))]
    # plain group 5 of row 1 decodes close to the gathered input
    deq = O.dequant(q, sf)
    assert deq.shape == (3, 4224)
    err = np.abs(deq[1, 80:96] - xg[1, 80:96].float().numpy())
    assert err.max() <= np.abs(xg[1, 80:96].float().numpy()).max() / 6 + 1e-6
    # critical group 0 = reordered channels 3968..3983: main at K_eff columns 3968..3983, residual next
    main = deq[:, 3968:3984]
    res = deq[:, 3984:4000]
    ref = xg[:, 3968:3984].float().numpy()
    assert np.abs(main + res - ref).max() < np.abs(main - ref).max() + 1e-9
    # never-written scale bytes keep the fill value
    written = np.zeros(sf.size, bool)
    written[O.sf_valid_offsets(3, kq + ke)] = True
    assert (sf[~written] == 0xEE).all()


def test_weight_residual_slot_is_a_copy_mode16_and_mode32():
    kq, ke = 256, 64
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(5, kq, generator=g)).to(torch.bfloat16)
    for mode in (16, 32):
        q, sf = O.quantize_w(w, None, ke, mode=mode)
        g0 = (kq - ke) // 16
        ncols = (kq + ke) // 16
        if mode == 16:
            for j in range(ke // 16):
                b = 8 * g0 + 16 * j
                assert (q[:, b:b + 8] == q[:, b + 8:b + 16]).all()
                for r in range(5):
                    assert sf[O.sf_offset(r, g0 + 2 * j, ncols)] == sf[O.sf_offset(r, g0 + 2 * j + 1, ncols)]
        else:
            for p in range(ke // 32):
                b = 8 * g0 + 32 * p
                assert (q[:, b:b + 16] == q[:, b + 16:b + 32]).all()
                for r in range(5):
                    for h in range(2):
                        assert sf[O.sf_offset(r, g0 + 4 * p + h, ncols)] == sf[O.sf_offset(r, g0 + 4 * p + h + 2, ncols)]


def test_mode32_differs_from_mode16_only_in_critical_region():
    kq, ke = 512, 64
    g = torch.Generator().manual_seed(2)
    x = (torch.randn(4, kq, generator=g) * 3).to(torch.bfloat16)
    q16, _ = O.quantize_x(x, None, ke, mode=16)
    q32, _ = O.quantize_x(x, None, ke, mode=32)
    plain = 8 * (kq - ke) // 16
    assert (q16[:, :plain] == q32[:, :plain]).all()
    # same main codes, re-ordered: [m0 r0 m1 r1] vs [m0 m1 r0 r1]
    assert (q16[:, plain:plain + 8] == q32[:, plain:plain + 8]).all()
    assert (q16[:, plain + 16:plain + 24] == q32[:, plain + 8:plain + 16]).all()
