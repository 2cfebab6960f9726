"""Writes tests/golden/transfers.npz: expected outputs of the CudaDMA transfer
rules on the inputs the reference's tests use (h_idata[i] = float(i),
src/tests/test_sequential/cudaDMA_test_sequential_v2.cu:417-418), computed with
plain numpy indexing -- independently of oracle/oracle.c, which the tests then
check against these vectors. The reference ships no stored vectors (its tests
recompute the expectation from the input), so these are the committed stand-in.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def strided_case(elmt_floats, rows, sstride_floats, dstride_floats, offset):
    src = np.arange(offset + (rows - 1) * sstride_floats + elmt_floats, dtype=np.float32)
    dst = np.zeros(offset + (rows - 1) * dstride_floats + elmt_floats, dtype=np.float32)
    for i in range(rows):
        dst[offset + i * dstride_floats: offset + i * dstride_floats + elmt_floats] = \
            src[offset + i * sstride_floats: offset + i * sstride_floats + elmt_floats]
    return dst


def gather_case(elmt_floats, index, pitch_floats):
    src = np.arange((max(index) + 1) * elmt_floats, dtype=np.float32)
    dst = np.zeros((len(index) - 1) * pitch_floats + elmt_floats, dtype=np.float32)
    for i, ix in enumerate(index):
        dst[i * pitch_floats: i * pitch_floats + elmt_floats] = src[ix * elmt_floats:(ix + 1) * elmt_floats]
    return dst


def scatter_case(elmt_floats, index, pitch_floats):
    src = np.arange((len(index) - 1) * pitch_floats + elmt_floats, dtype=np.float32) + 1
    dst = np.zeros((max(index) + 1) * elmt_floats, dtype=np.float32)
    for i, ix in enumerate(index):
        dst[ix * elmt_floats:(ix + 1) * elmt_floats] = src[i * pitch_floats: i * pitch_floats + elmt_floats]
    return dst


def halo_case(dimx, dimy, pitch, radius, corners):
    src = (np.arange(pitch * (dimy + 2 * radius), dtype=np.float32) % 97 + 1).reshape(dimy + 2 * radius, pitch)
    dst = np.zeros((dimy + 2 * radius, dimx + 2 * radius), dtype=np.float32)
    w = dimx + 2 * radius
    x0, x1 = (0, w) if corners else (radius, radius + dimx)
    dst[:radius, x0:x1] = src[:radius, x0:x1]
    dst[radius + dimy:, x0:x1] = src[radius + dimy:, x0:x1]
    dst[radius:radius + dimy, :radius] = src[radius:radius + dimy, :radius]
    dst[radius:radius + dimy, radius + dimx:w] = src[radius:radius + dimy, radius + dimx:w]
    return dst.ravel()


def stencil_case(nx, ny, nz, steps, coeff):
    u = ((np.arange(nx * ny * nz) * 2654435761 % 1000) / 1000.0).astype(np.float32).astype(np.float64).reshape(nz, ny, nx)
    c = [float(np.float32(v)) for v in coeff]
    for _ in range(steps):
        p = np.pad(u, 4)
        out = c[0] * u
        for r in range(1, 5):
            out = out + c[r] * (p[4 - r:4 - r + nz, 4:-4, 4:-4] + p[4 + r:4 + r + nz, 4:-4, 4:-4] +
                                p[4:-4, 4 - r:4 - r + ny, 4:-4] + p[4:-4, 4 + r:4 + r + ny, 4:-4] +
                                p[4:-4, 4:-4, 4 - r:4 - r + nx] + p[4:-4, 4:-4, 4 + r:4 + r + nx])
        u = out
    return u.astype(np.float32).ravel()


def main():
    out = {}
    # splitmix64: the generator's published first outputs for seed 0 (state advances by the golden-ratio increment)
    out["splitmix64_seed0"] = np.array([0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F], dtype=np.uint64)
    out["strided_a"] = strided_case(64, 128, 16384, 64, 0)
    out["strided_b"] = strided_case(25, 7, 33, 26, 1)
    out["strided_c"] = strided_case(80, 24, 1024, 80, 0)
    idx = [5, 0, 17, 3, 9, 31, 2, 11]
    out["index"] = np.array(idx, dtype=np.int32)
    out["gather_packed"] = gather_case(8, idx, 8)
    out["gather_pitched"] = gather_case(3, idx, 5)
    out["scatter_packed"] = scatter_case(8, idx, 8)
    out["scatter_pitched"] = scatter_case(3, idx, 5)
    out["halo_r4_nocorners"] = halo_case(32, 16, 64, 4, False)
    out["halo_r4_corners"] = halo_case(32, 16, 64, 4, True)
    out["halo_r1_corners"] = halo_case(9, 11, 20, 1, True)
    out["halo_r8_nocorners"] = halo_case(17, 8, 40, 8, False)
    coeff = (-2.847, 1.6, -0.2, 0.0254, -0.00179)
    out["stencil_12x10x9_s2"] = stencil_case(12, 10, 9, 2, coeff)
    out["stencil_5x4x3_s1"] = stencil_case(5, 4, 3, 1, coeff)
    np.savez_compressed(os.path.join(HERE, "transfers.npz"), **out)
    print("wrote", os.path.join(HERE, "transfers.npz"), sum(v.nbytes for v in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
