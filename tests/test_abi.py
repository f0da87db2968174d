"""CPU tests of the C-ABI library: it loads, exports every symbol the header declares, its structs have the layout
the Python mirror assumes, and its host-only entry points (validation, resize parameters) behave.  No compute call
is made here (there is no GPU)."""
import ctypes as C
import os
import re
import subprocess
import tempfile

import numpy as np
import pytest

import oracle
from conftest import ROOT
from fusedkernellibrary_b200 import abi, workloads as W

HEADER = os.path.join(ROOT, "include", "fkb", "fkb.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fkb_[a-z_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = abi.load()
    names = declared_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in fkb.h but not exported"
        assert n in abi.SIGNATURES, f"{n} has no ctypes signature"
    assert lib.fkb_abi_version() == 3


def test_struct_layout_matches_header():
    prog = r'''
    #include <stdio.h>
    #include <stddef.h>
    #include "fkb/fkb.h"
    int main(void) {
      printf("%zu %zu %zu ", sizeof(fkb_op), sizeof(fkb_chain_desc), sizeof(fkb_plane_desc));
      printf("%zu %zu %zu %zu %zu %zu %zu\n", offsetof(fkb_chain_desc, ops), offsetof(fkb_chain_desc, ccm),
             offsetof(fkb_plane_desc, dst_channel_stride), offsetof(fkb_plane_desc, fx), offsetof(fkb_plane_desc, bg),
             offsetof(fkb_plane_desc, chain), offsetof(fkb_plane_desc, params));
      return 0; }'''
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.c")
        open(src, "w").write(prog)
        subprocess.run(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), src, "-o", os.path.join(d, "t")], check=True)
        out = subprocess.run([os.path.join(d, "t")], check=True, capture_output=True, text=True).stdout.split()
    got = [int(v) for v in out]
    want = [C.sizeof(abi.Op), C.sizeof(abi.ChainDesc), C.sizeof(abi.PlaneDesc), abi.ChainDesc.ops.offset, abi.ChainDesc.ccm.offset,
            abi.PlaneDesc.dst_channel_stride.offset, abi.PlaneDesc.fx.offset, abi.PlaneDesc.bg.offset, abi.PlaneDesc.chain.offset,
            abi.PlaneDesc.params.offset]
    assert got == want


def test_resize_params_match_oracle():
    lib, orc = abi.load(), oracle.load_oracle()
    rs = np.random.RandomState(2)
    for _ in range(5000):
        sw, sh, dw, dh = (int(v) for v in rs.randint(1, 2000, 4))
        for geom in (abi.GEOM_RESIZE_IGNORE_AR, abi.GEOM_RESIZE_PRESERVE_AR, abi.GEOM_RESIZE_PRESERVE_AR_RN_EVEN, abi.GEOM_RESIZE_PRESERVE_AR_LEFT):
            a, b = abi.PlaneDesc(), abi.PlaneDesc()
            for d in (a, b):
                d.crop_w, d.crop_h, d.dst_w, d.dst_h = sw, sh, dw, dh
            assert lib.fkb_resize_params(geom, C.byref(a)) == 0 and orc.fkb_oracle_resize_params(geom, C.byref(b)) == 0
            assert (a.fx, a.fy, a.x1, a.y1, a.x2, a.y2) == (b.fx, b.fy, b.x1, b.y1, b.x2, b.y2), (sw, sh, dw, dh, geom)
    bad = abi.PlaneDesc()
    assert lib.fkb_resize_params(abi.GEOM_RESIZE_IGNORE_AR, C.byref(bad)) == abi.ERR_INVALID
    assert lib.fkb_resize_params(abi.GEOM_RESIZE_IGNORE_AR, None) == abi.ERR_NULL


def test_ycbcr_matrices_match_oracle():
    lib, orc = abi.load(), oracle.load_oracle()
    for rng in (abi.RANGE_LIMITED, abi.RANGE_FULL):
        for prim in (abi.PRIMITIVES_BT601, abi.PRIMITIVES_BT709, abi.PRIMITIVES_BT2020):
            a, b, sa, sb = (C.c_float * 9)(), (C.c_float * 9)(), (C.c_float * 3)(), (C.c_float * 3)()
            assert lib.fkb_ycbcr_to_rgb(rng, prim, a, sa) == 0 and orc.fkb_oracle_ycbcr_to_rgb(rng, prim, b, sb) == 0
            assert list(a) == list(b) and list(sa) == list(sb)
    assert lib.fkb_ycbcr_to_rgb(2, 0, a, sa) == abi.ERR_INVALID and lib.fkb_ycbcr_to_rgb(0, 3, a, sa) == abi.ERR_INVALID
    assert lib.fkb_ycbcr_to_rgb(0, 0, None, sa) == abi.ERR_NULL
    for rng in (abi.RANGE_LIMITED, abi.RANGE_FULL):
        for prim in (abi.PRIMITIVES_BT601, abi.PRIMITIVES_BT709, abi.PRIMITIVES_BT2020):
            assert lib.fkb_rgb_to_ycbcr(rng, prim, a, sa) == 0 and orc.fkb_oracle_rgb_to_ycbcr(rng, prim, b, sb) == 0
            assert list(a) == list(b) and list(sa) == list(sb)


def _bound(wl):
    """Planes bound to fake, well-aligned addresses: enough for the host-only validator."""
    return wl.bind([0x10000000 + i * 0x10000000 for i in range(len(wl.sources))],
                   [0x7000000000 + i * 0x100000000 for i in range(len(wl.out_sizes))])


@pytest.mark.parametrize("factory,kw", [
    (W.readme_crops, {}), (W.vertical_fusion, {"w": 64, "h": 8}), (W.nv12_preprocess, {"w": 64, "h": 36, "dst": (32, 32)}),
    (W.batched_crop_resize, {"n_frames": 2, "crops_per_frame": 2, "w": 320, "h": 200}), (W.divergent_planes, {"n_per_seq": 2, "w": 64, "h": 36}),
])
def test_validate_accepts_the_configurations(factory, kw):
    wl = factory(**kw)
    assert abi.load().fkb_validate(wl.chain_array(), len(wl.chains), _bound(wl), len(wl.planes)) == abi.OK


def test_validate_rejects_bad_descriptors():
    lib = abi.load()
    wl = W.readme_crops()
    chains, n = wl.chain_array(), len(wl.planes)

    def status(mutate, chains_=None):
        planes = _bound(wl)
        ch = chains_ if chains_ is not None else wl.chain_array()
        mutate(planes, ch)
        return lib.fkb_validate(ch, 1, planes, n)

    assert lib.fkb_validate(None, 1, _bound(wl), n) == abi.ERR_NULL
    assert lib.fkb_validate(chains, 1, None, n) == abi.ERR_NULL
    assert lib.fkb_validate(chains, 1, _bound(wl), 0) == abi.ERR_INVALID          # no planes
    assert lib.fkb_validate(chains, 0, _bound(wl), n) == abi.ERR_INVALID          # no chains
    assert lib.fkb_validate(chains, abi.MAX_CHAINS + 1, _bound(wl), n) == abi.ERR_INVALID
    assert status(lambda p, c: setattr(p[1], "src", None)) == abi.ERR_NULL
    assert status(lambda p, c: setattr(p[2], "dst", None)) == abi.ERR_NULL
    assert status(lambda p, c: setattr(p[0], "src_pitch", 1920 * 3 - 1)) == abi.ERR_INVALID   # pitch < row
    assert status(lambda p, c: setattr(p[0], "crop_x", 1900)) == abi.ERR_INVALID              # rect leaves the frame
    assert status(lambda p, c: setattr(p[0], "crop_h", 0)) == abi.ERR_INVALID
    assert status(lambda p, c: setattr(p[0], "crop_w", -4)) == abi.ERR_INVALID
    assert status(lambda p, c: setattr(p[3], "dst_pitch", 128 * 3 - 1)) == abi.ERR_INVALID
    assert status(lambda p, c: setattr(p[3], "fx", 0.0)) == abi.ERR_INVALID
    assert status(lambda p, c: setattr(p[3], "fy", float("nan"))) == abi.ERR_INVALID
    # source coordinates of 2^22 and more (fx * dst_w) are refused: the kernels take floors without a conversion
    assert status(lambda p, c: setattr(p[3], "fx", float(2 ** 22) / p[3].dst_w)) == abi.ERR_UNSUPPORTED
    assert status(lambda p, c: setattr(p[3], "fy", float(2 ** 21) / p[3].dst_h)) == abi.OK
    assert status(lambda p, c: setattr(p[4], "x2", 128)) == abi.ERR_INVALID                   # letterbox outside dst
    assert status(lambda p, c: setattr(p[4], "chain", 1)) == abi.ERR_INVALID                  # chain index out of range
    assert status(lambda p, c: setattr(c[0], "dst_format", abi.PIX_F32C3)) == abi.ERR_INVALID  # chain ends in uchar3
    assert status(lambda p, c: setattr(c[0], "n_ops", abi.MAX_OPS + 1)) == abi.ERR_INVALID
    assert status(lambda p, c: setattr(c[0], "src_format", 12)) == abi.ERR_UNSUPPORTED
    assert status(lambda p, c: setattr(c[0].ops[0], "code", 77)) == abi.ERR_UNSUPPORTED
    assert status(lambda p, c: setattr(c[0].ops[0], "plane_slot", 4)) == abi.ERR_INVALID

    # type flow: Mul<float3> straight after a uchar3 read is ill-typed (a compile error in the reference)
    bad = W.chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C3, abi.WRITE_PACKED, [W.op(abi.OP_MUL, (2, 2, 2))])
    wl2 = W.vertical_fusion(w=32, h=4)
    arr = (abi.ChainDesc * 1)(bad)
    assert lib.fkb_validate(arr, 1, _bound(wl2), 1) == abi.ERR_INVALID
    # AddOpaqueAlpha: once, and only on the way from a three-channel source to a four-channel write
    wl4 = W.add_alpha_image(w=32, h=4)
    assert lib.fkb_validate(wl4.chain_array(), 1, _bound(wl4), 1) == abi.OK
    two = W.chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C4, abi.WRITE_PACKED, [W.op(abi.OP_ADD_ALPHA, (255, 0, 0))] * 2)
    assert lib.fkb_validate((abi.ChainDesc * 1)(two), 1, _bound(wl4), 1) == abi.ERR_INVALID
    none = W.chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C4, abi.WRITE_PACKED, [])
    assert lib.fkb_validate((abi.ChainDesc * 1)(none), 1, _bound(wl4), 1) == abi.ERR_INVALID
    three = W.chain(abi.PIX_U8C3, abi.GEOM_NONE, abi.PIX_U8C3, abi.WRITE_PACKED, [W.op(abi.OP_ADD_ALPHA, (255, 0, 0))])
    assert lib.fkb_validate((abi.ChainDesc * 1)(three), 1, _bound(wl2), 1) == abi.ERR_INVALID
    # geometry NONE cannot write more pixels than the crop holds
    wl3 = W.crop_reorder(n=1)
    p3 = _bound(wl3)
    p3[0].dst_w = p3[0].crop_w + 1
    p3[0].dst_pitch = (p3[0].crop_w + 1) * 3
    assert lib.fkb_validate(wl3.chain_array(), 1, p3, 1) == abi.ERR_INVALID


def test_launch_rejects_before_touching_the_device():
    # invalid launches are refused on the host: no CUDA call is made, so this runs without a GPU
    lib = abi.load()
    wl = W.readme_crops()
    planes = _bound(wl)
    planes[0].src = None
    assert lib.fkb_launch_transform(wl.chain_array(), planes, len(wl.planes), None) == abi.ERR_NULL
    assert lib.fkb_launch_transform(None, planes, 1, None) == abi.ERR_NULL
    assert lib.fkb_launch_divergent(wl.chain_array(), 1, planes, 0, None) == abi.ERR_INVALID
    assert lib.fkb_plan_launch(None, None) == abi.ERR_NULL
    out = C.c_void_p()
    assert lib.fkb_plan_create(wl.chain_array(), 1, planes, len(wl.planes), C.byref(out)) == abi.ERR_NULL and not out.value
    assert lib.fkb_status_string(abi.ERR_UNSUPPORTED) == b"unsupported chain"


def test_algorithmic_bytes_closed_forms():
    assert W.vertical_fusion().algorithmic_bytes()["total"] == 49_766_400
    assert W.divergent_planes(n_per_seq=1, w=384, h=216).algorithmic_bytes()["total"] == (384 * 216 * 3 + 192 * 108 * 3) + (384 * 216 * 15)
    rc = W.readme_crops().algorithmic_bytes()
    assert rc["dst"] == 122_880 and 60_000 < rc["src"] < 80_000
