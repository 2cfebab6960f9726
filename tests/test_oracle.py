"""The CPU oracle against the committed golden vectors (tests/golden, made by an
independent numpy restatement) and against properties of the rules it restates.
Runs without a GPU."""
import os

import numpy as np
import pytest

from oracle import oracle

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "transfers.npz"))
COEFF = (-2.847, 1.6, -0.2, 0.0254, -0.00179)


def test_splitmix64_known_answers():
    inc = 0x9E3779B97F4A7C15
    got = [oracle.lib().oracle_splitmix64((i * inc) & (2**64 - 1)) for i in range(3)]
    assert got == [int(v) for v in GOLD["splitmix64_seed0"]]


def test_fills_are_seeded_and_in_range():
    a = oracle.fill_uniform(10000, 0xC1, -1.0, 1.0)
    assert np.array_equal(a, oracle.fill_uniform(10000, 0xC1, -1.0, 1.0))
    assert a.min() >= -1.0 and a.max() < 1.0 and abs(a.mean()) < 0.05
    assert not np.array_equal(a, oracle.fill_uniform(10000, 0xC2, -1.0, 1.0))
    # element i depends on seed + i only: a shifted seed gives the shifted sequence
    assert np.array_equal(a[5:], oracle.fill_uniform(10000 - 5, 0xC1 + 5, -1.0, 1.0))
    idx = oracle.fill_index(10000, 0xC3A, 1 << 24)
    assert idx.min() >= 0 and idx.max() < (1 << 24)
    p = oracle.permutation(4096, 0xC3B)
    assert np.array_equal(np.sort(p), np.arange(4096))
    assert np.array_equal(oracle.permutation(1, 7), [0])
    assert oracle.permutation(0, 7).size == 0


@pytest.mark.parametrize("name,elmt,rows,ss,ds,off", [("strided_a", 64, 128, 16384, 64, 0), ("strided_b", 25, 7, 33, 26, 1),
                                                      ("strided_c", 80, 24, 1024, 80, 0)])
def test_strided_golden(name, elmt, rows, ss, ds, off):
    src = np.arange(off + (rows - 1) * ss + elmt, dtype=np.float32)
    dst = np.zeros(GOLD[name].size, dtype=np.float32)
    oracle.strided(dst[off:].view(np.uint8), src[off:].view(np.uint8), elmt * 4, rows, ss * 4, ds * 4)
    assert np.array_equal(dst, GOLD[name])


def test_sequential_and_empty_transfers():
    src = np.arange(1000, dtype=np.float32)
    assert np.array_equal(oracle.sequential(src).view(np.float32), src)
    dst = np.full(16, 7, dtype=np.uint8)
    oracle.strided(dst, dst.copy(), 4, 0, 8, 4)  # zero rows: nothing moves
    assert (dst == 7).all()
    assert oracle.sequential(np.zeros(0, dtype=np.float32)).size == 0


@pytest.mark.parametrize("name,elmt,pitch", [("gather_packed", 8, 8), ("gather_pitched", 3, 5)])
def test_gather_golden(name, elmt, pitch):
    idx = GOLD["index"]
    src = np.arange((idx.max() + 1) * elmt, dtype=np.float32)
    dst = np.zeros(GOLD[name].size, dtype=np.float32)
    oracle.gather(dst.view(np.uint8), src.view(np.uint8), idx, elmt * 4, pitch * 4 if pitch != elmt else 0)
    assert np.array_equal(dst, GOLD[name])


@pytest.mark.parametrize("name,elmt,pitch", [("scatter_packed", 8, 8), ("scatter_pitched", 3, 5)])
def test_scatter_golden_and_inverse(name, elmt, pitch):
    idx = GOLD["index"]
    src = np.arange((idx.size - 1) * pitch + elmt, dtype=np.float32) + 1
    dst = np.zeros(GOLD[name].size, dtype=np.float32)
    alt = pitch * 4 if pitch != elmt else 0
    oracle.scatter(dst.view(np.uint8), src.view(np.uint8), idx, elmt * 4, alt)
    assert np.array_equal(dst, GOLD[name])
    # gathering with the same indices undoes the scatter on the rows that were moved
    back = np.zeros_like(src)
    oracle.gather(back.view(np.uint8), dst.view(np.uint8), idx, elmt * 4, alt)
    for i in range(idx.size):
        assert np.array_equal(back[i * pitch:i * pitch + elmt], src[i * pitch:i * pitch + elmt])


@pytest.mark.parametrize("name,dimx,dimy,pitch,radius,corners",
                         [("halo_r4_nocorners", 32, 16, 64, 4, 0), ("halo_r4_corners", 32, 16, 64, 4, 1),
                          ("halo_r1_corners", 9, 11, 20, 1, 1), ("halo_r8_nocorners", 17, 8, 40, 8, 0)])
def test_halo_golden(name, dimx, dimy, pitch, radius, corners):
    src = (np.arange(pitch * (dimy + 2 * radius), dtype=np.float32) % 97 + 1)
    dst = np.zeros(GOLD[name].size, dtype=np.float32)
    oracle.halo_ring(dst.view(np.uint8), src.view(np.uint8), dimx, dimy, pitch, radius, corners, 4)
    assert np.array_equal(dst, GOLD[name])
    # wider elements are the same rule on wider cells
    src2 = np.repeat(src, 2)
    dst2 = np.zeros(dst.size * 2, dtype=np.float32)
    oracle.halo_ring(dst2.view(np.uint8), src2.view(np.uint8), dimx, dimy, pitch, radius, corners, 8)
    assert np.array_equal(dst2, np.repeat(GOLD[name], 2))


def test_workload_restatements():
    src = oracle.fill_uniform(16384 * 5 // 4 + 100, 0xC1, -1.0, 1.0)
    assert np.array_equal(oracle.chunked_copy(src, 16384), src)
    m = oracle.fill_uniform(256 * 192, 0xC2, -1.0, 1.0).reshape(256, 192)
    assert np.array_equal(oracle.tile_transpose(m), m.T)
    assert np.array_equal(oracle.tile_transpose(m[:130, :70]), m[:130, :70].T)  # ragged tiles
    table = oracle.fill_uniform(512 * 8, 0xC3, -1.0, 1.0)
    g = oracle.fill_index(256, 0xC3A, 512)
    s = oracle.permutation(256, 0xC3B)
    out = oracle.gather_scatter(np.zeros(256 * 8, dtype=np.float32), table, g, s)
    assert np.array_equal(out.reshape(256, 8)[s], table.reshape(512, 8)[g])


@pytest.mark.parametrize("name,nx,ny,nz,steps", [("stencil_12x10x9_s2", 12, 10, 9, 2), ("stencil_5x4x3_s1", 5, 4, 3, 1)])
def test_stencil_golden(name, nx, ny, nz, steps):
    u = ((np.arange(nx * ny * nz) * 2654435761 % 1000) / 1000.0).astype(np.float32).reshape(nz, ny, nx)
    got = oracle.stencil25_f64(u, COEFF, steps).ravel()
    assert np.array_equal(got, GOLD[name])


def test_stencil_fp32_baseline_tracks_the_double_oracle():
    f = oracle.fill_uniform(40 * 24 * 20, 0xC4, 0.0, 1.0).reshape(20, 24, 40)
    a = oracle.stencil25_f64(f, COEFF, 1)
    b = oracle.stencil25_step_f32(f, COEFF)
    assert np.abs(a - b).max() / np.abs(a).max() < 1e-6
    # a constant interior field maps to the coefficient sum away from the faces
    c = np.ones((20, 24, 40), dtype=np.float32)
    s = oracle.stencil25_f64(c, COEFF, 1)
    total = COEFF[0] + 6 * sum(COEFF[1:])
    assert abs(s[10, 12, 20] - total) < 1e-5
