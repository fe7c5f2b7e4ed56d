"""Device memory mapped on demand (qb_pool_*, qb_region_*: the reference's src/cuda/vmm.rs): budget accounting, pages
zeroed when mapped and reused when unmapped, partial unmaps, refused accesses to ranges that are not mapped (no access
to an unmapped page is ever made), and a kernel of the library working on a mapped region."""
import numpy as np
import pytest
import torch

from qwenny_b200 import vmm
from qwenny_b200._lib import QbError

pytestmark = pytest.mark.gpu


def test_pool_and_regions(ctx):
    pool = vmm.Pool(0)
    pg = pool.page
    assert pg >= 1 << 16 and pg & (pg - 1) == 0
    pool.set_budget(6)
    a, b = vmm.Region(pool, 5 * pg - 100), vmm.Region(pool, 4 * pg)
    assert a.size == 5 * pg and b.size == 4 * pg and a.ptr and b.ptr and a.ptr != b.ptr
    assert pool.usage() == (0, 6) and pool.available() == 6
    assert a.map(0, 3 * pg) and pool.usage() == (3, 6)
    assert a.is_mapped(0, 3 * pg) and not a.is_mapped(0, 3 * pg + 1)
    assert not a.read(pg - 64, 4096).any()  # zeroed
    pat = (np.arange(3 * pg, dtype=np.uint32) * 2654435761 >> 13).astype(np.uint8)
    a.write(0, pat)
    assert np.array_equal(a.read(0, 3 * pg), pat)
    # too few pages left: nothing more is mapped
    assert not b.map(0, 4 * pg) and not b.is_mapped(0, 1) and pool.usage() == (3, 6)
    assert b.map(pg, 4 * pg) and pool.usage() == (6, 6) and pool.available() == 0
    assert not a.map(3 * pg, 4 * pg)
    # ranges that are not mapped are refused, not touched
    with pytest.raises(QbError):
        a.read(3 * pg - 8, 16)
    with pytest.raises(QbError):
        b.write(0, np.zeros(8, dtype=np.uint8))
    with pytest.raises(QbError):
        a.read(5 * pg - 8, 16)  # beyond the region
    # only the pages wholly inside the range go
    a.unmap(pg // 2, 2 * pg + pg // 2)
    assert a.is_mapped(0, pg) and not a.is_mapped(pg, 2 * pg) and a.is_mapped(2 * pg, 3 * pg)
    assert pool.usage() == (5, 6) and pool.available() == 1
    assert np.array_equal(a.read(0, pg), pat[:pg]) and np.array_equal(a.read(2 * pg, pg), pat[2 * pg:])
    # the freed page comes back zeroed
    assert a.map(pg, 2 * pg) and pool.usage() == (6, 6)
    assert not a.read(pg, pg).any()
    # pages given back to the driver lower the budget
    b.unmap(0, 4 * pg)
    assert pool.usage() == (3, 6) and pool.release(2) == 2 and pool.usage() == (3, 4) and pool.available() == 1
    pool.set_budget(5)
    pool.fill()
    assert pool.usage() == (3, 5) and pool.available() == 2
    a.close()
    b.close()
    assert pool.usage()[0] == 0
    pool.close()


def test_a_kernel_on_a_mapped_region(ctx):
    """The library's kernels take a region's fixed address like any device pointer: f32 -> f16 conversion (qb_to_xin)
    of rows written through the region, before and after the region grows."""
    pool = vmm.Pool(0)
    pg = pool.page
    r = vmm.Region(pool, 8 * pg)
    assert r.map(0, pg)
    g = np.random.default_rng(0)
    x = g.standard_normal(pg // 4).astype(np.float32)
    r.write(0, x)
    y = torch.zeros(pg // 4, dtype=torch.float16, device="cuda")
    ctx.to_xin(r.ptr, y, pg // 4)
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy(), x.astype(np.float16))
    # grow: the address of the first page does not move, its content stays
    assert r.map(pg, 3 * pg)
    x2 = g.standard_normal(3 * pg // 4).astype(np.float32)
    r.write(pg, x2[pg // 4:])
    y2 = torch.zeros(3 * pg // 4, dtype=torch.float16, device="cuda")
    ctx.to_xin(r.ptr, y2, 3 * pg // 4)
    torch.cuda.synchronize()
    want = np.concatenate([x, x2[pg // 4:]]).astype(np.float16)
    assert np.array_equal(y2.cpu().numpy(), want)
    r.close()
    pool.close()
