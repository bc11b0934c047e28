"""Operand-encoding self-test of the tensor path: a caller-built shared-memory image, explicit descriptors, and
the raw accumulator compared with a plain matrix product.  Pins the two layout conventions the kernels rely on:
  * K-major operands with the 128-byte swizzle (SDDMM: gathered rhs rows and lhs rows), and
  * MN-major operands — A with the 128-byte swizzle, B unswizzled — (SpMM: gathered rows of the dense operand
    and the value vectors)."""
import ctypes as C

import numpy as np
import pytest
import torch

from vectorsparse_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def desc(start, lbo, sbo, swizzle):
    return (start >> 4) | ((lbo >> 4) << 16) | ((sbo >> 4) << 32) | (1 << 46) | (swizzle << 61)


def idesc(M, N, a_mn, b_mn):
    return (1 << 4) | (a_mn << 15) | (b_mn << 16) | ((N >> 3) << 17) | ((M >> 4) << 24)


def run(image, descs, idesc_, ncols):
    img = torch.from_numpy(image.view(np.uint8)).to("cuda:0")
    d = np.array(descs, dtype=np.uint64)   # host array: the library checks every descriptor against the image
    out = torch.zeros(128 * ncols, dtype=torch.float32, device="cuda:0")
    rc = _lib.lib().vs_selftest_mma(img.data_ptr(), img.numel(), d.ctypes.data, len(descs) // 2, idesc_, ncols,
                                    -77.0, out.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return out.cpu().numpy().reshape(128, ncols)


def put(image, byte_off, value):
    image[byte_off // 2] = value


def test_k_major_swizzle128():
    rng = np.random.default_rng(0)
    A = rng.integers(-4, 5, (128, 64)).astype(np.float16)
    B = rng.integers(-4, 5, (16, 64)).astype(np.float16)
    image = np.zeros((16384 + 2048) // 2, np.float16)
    for (mat, base, rows) in ((A, 0, 128), (B, 16384, 16)):
        for r in range(rows):
            for kk in range(64):
                off = base + (r // 8) * 1024 + (r % 8) * 128 + (((kk // 8) ^ (r % 8)) * 16) + (kk % 8) * 2
                put(image, off, mat[r, kk])
    descs = []
    for mm in range(4):
        descs += [desc(mm * 32, 16, 1024, 2), desc(16384 + mm * 32, 16, 1024, 2)]
    got = run(image, descs, idesc(128, 16, 0, 0), 16)
    want = A.astype(np.float32) @ B.astype(np.float32).T
    assert np.array_equal(got, want)


def test_mn_major_spmm_layout():
    rng = np.random.default_rng(1)
    KK = 32
    A = rng.integers(-4, 5, (128, KK)).astype(np.float16)   # [dense column m][nonzero kk]
    B = rng.integers(-4, 5, (KK, 16)).astype(np.float16)    # [nonzero kk][vector element nn]
    a_bytes, v_base, z_off = 8192, 8192, 1024
    image = np.zeros((a_bytes + 2048) // 2, np.float16)
    for m in range(128):
        for kk in range(KK):
            off = (m // 64) * 4096 + (kk // 8) * 1024 + (kk % 8) * 128 + ((((m % 64) // 8) ^ (kk % 8)) * 16) + (m % 8) * 2
            put(image, off, A[m, kk])
    for kk in range(KK):
        for nn in range(16):
            off = v_base + (nn // 8) * z_off + kk * 16 + (nn % 8) * 2
            put(image, off, B[kk, nn])
    descs = []
    for mm in range(KK // 16):
        descs += [desc(mm * 2048, 4096, 1024, 2), desc(v_base + mm * 256, 128, z_off, 0)]
    got = run(image, descs, idesc(128, 16, 1, 1), 16)
    want = A.astype(np.float32) @ B.astype(np.float32)
    assert np.array_equal(got, want)


def test_tma_row_gather4():
    """Four-row hardware gathers: rows land consecutively, 128 bytes each, 16-byte chunks XOR-swizzled with the
    row's position inside its 1024-byte block; rows outside the matrix arrive as zeros."""
    rng = np.random.default_rng(2)
    rows, cols, groups, x = 50, 192, 6, 64
    mat = rng.integers(-100, 100, (rows, cols)).astype(np.float16)
    idx = rng.integers(0, rows, 4 * groups).astype(np.int32)
    idx[5] = rows          # out of range: zero fill
    idx[10] = rows + 7
    d_mat = torch.from_numpy(mat).to("cuda:0")
    d_idx = torch.from_numpy(idx).to("cuda:0")
    out = torch.zeros(groups * 512, dtype=torch.uint8, device="cuda:0")
    rc = _lib.lib().vs_selftest_gather4(d_mat.data_ptr(), rows, cols, d_idx.data_ptr(), groups, x, out.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = out.cpu().numpy().view(np.float16).reshape(groups * 4, 8, 8)   # [row slot][16-byte chunk][8 halves]
    for slot in range(groups * 4):
        src = mat[idx[slot], x:x + 64].reshape(8, 8) if idx[slot] < rows else np.zeros((8, 8), np.float16)
        for c in range(8):
            assert np.array_equal(got[slot, c ^ (slot % 8)], src[c]), (slot, c)


def test_mn_major_both_swizzled_wide():
    """Densified SpMM: A MN-major (128 rows of the sparse tile contiguous, two 64-row atoms 8 KiB apart), B
    MN-major (64-row x 64-column boxes of the dense operand as TMA writes them, one box per 64 columns, 8 KiB
    apart), both with the 128-byte swizzle, N = 128, four K = 16 steps 2 KiB apart."""
    rng = np.random.default_rng(3)
    KK, NN = 64, 128
    A = rng.integers(-4, 5, (128, KK)).astype(np.float16)
    B = rng.integers(-4, 5, (KK, NN)).astype(np.float16)
    b_base = 16384
    image = np.zeros((b_base + 2 * 8192) // 2, np.float16)
    for m in range(128):
        for kk in range(KK):
            off = (m // 64) * 8192 + (kk // 8) * 1024 + (kk % 8) * 128 + ((((m % 64) // 8) ^ (kk % 8)) * 16) + (m % 8) * 2
            put(image, off, A[m, kk])
    for kk in range(KK):
        for n in range(NN):
            off = b_base + (n // 64) * 8192 + (kk // 8) * 1024 + (kk % 8) * 128 + ((((n % 64) // 8) ^ (kk % 8)) * 16) + (n % 8) * 2
            put(image, off, B[kk, n])
    descs = []
    for mm in range(KK // 16):
        descs += [desc(mm * 2048, 8192, 1024, 2), desc(b_base + mm * 2048, 8192, 1024, 2)]
    got = run(image, descs, idesc(128, NN, 1, 1), NN)
    want = A.astype(np.float32) @ B.astype(np.float32)
    assert np.array_equal(got, want)


def test_pair_of_ctas_m256_n256():
    """Two CTAs, one MMA stream (cta_group::2, M = 256, N = 256): CTA r holds rows 128 r .. of A and of the
    accumulator and columns 128 r .. of B; operands in the densified-SpMM layouts (both MN-major, 128-byte swizzle),
    four K = 16 steps.  Also pins that the issuing CTA can tell the other CTA's barrier with a commit of its own."""
    rng = np.random.default_rng(4)
    KK, NN = 64, 256
    A = rng.integers(-4, 5, (256, KK)).astype(np.float16)
    B = rng.integers(-4, 5, (KK, NN)).astype(np.float16)
    b_base = 16384
    images = []
    for r in range(2):
        image = np.zeros((b_base + 2 * 8192) // 2, np.float16)
        Ar, Br = A[128 * r:128 * r + 128], B[:, 128 * r:128 * r + 128]
        for m in range(128):
            for kk in range(KK):
                off = (m // 64) * 8192 + (kk // 8) * 1024 + (kk % 8) * 128 + ((((m % 64) // 8) ^ (kk % 8)) * 16) + (m % 8) * 2
                put(image, off, Ar[m, kk])
        for kk in range(KK):
            for n in range(128):
                off = b_base + (n // 64) * 8192 + (kk // 8) * 1024 + (kk % 8) * 128 + ((((n % 64) // 8) ^ (kk % 8)) * 16) + (n % 8) * 2
                put(image, off, Br[kk, n])
        images.append(torch.from_numpy(image.view(np.uint8)).to("cuda:0"))
    descs = []
    for mm in range(KK // 16):
        descs += [desc(mm * 2048, 8192, 1024, 2), desc(b_base + mm * 2048, 8192, 1024, 2)]
    d = np.array(descs, dtype=np.uint64)
    out = torch.zeros(256 * NN, dtype=torch.float32, device="cuda:0")
    rc = _lib.lib().vs_selftest_mma_pair(images[0].data_ptr(), images[1].data_ptr(), images[0].numel(), d.ctypes.data,
                                         len(descs) // 2, idesc(256, NN, 1, 1), NN, -77.0, out.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = out.cpu().numpy().reshape(256, NN)
    want = A.astype(np.float32) @ B.astype(np.float32)
    assert np.array_equal(got, want)


def test_descriptors_outside_the_image_are_refused():
    """An operand that would reach past the image is rejected on the host: nothing is launched."""
    image = torch.zeros(16384 + 2048, dtype=torch.uint8, device="cuda:0")
    out = torch.zeros(128 * 16, dtype=torch.float32, device="cuda:0")
    L = _lib.lib()

    def rc(descs, idesc_, ncols=16):
        d = np.array(descs, dtype=np.uint64)
        return L.vs_selftest_mma(image.data_ptr(), image.numel(), d.ctypes.data, len(descs) // 2, idesc_, ncols, 0.0,
                                 out.data_ptr(), None)

    good = [desc(0, 16, 1024, 2), desc(16384, 16, 1024, 2)]
    assert rc(good, idesc(128, 16, 0, 0)) == 0
    assert rc([desc(4096, 16, 1024, 2), good[1]], idesc(128, 16, 0, 0)) == -3    # A: 16 blocks of 1 KiB from 4096 > image
    assert rc([good[0], desc(16384, 16, 8192, 2)], idesc(128, 16, 0, 0)) == -3   # B: second block 8 KiB on
    assert rc(good, idesc(128, 32, 0, 0), 16) == -3                              # N wider than the accumulator columns read
    assert rc(good, idesc(64, 16, 0, 0)) == -3                                   # M the sandbox does not run
    assert rc([desc(0, 16, 1024, 4), good[1]], idesc(128, 16, 0, 0)) == -3       # a swizzle mode no kernel uses
    torch.cuda.synchronize()
    assert ops.device_status() == 0
