"""The C-ABI library loads without a GPU and exports every symbol the header declares (no compute calls here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    from qvb8_b200 import build
    return build.build()


def _declared():
    names = []
    for h in os.listdir(os.path.join(ROOT, "include")):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(qvb8r?_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_builds_and_exports_header_symbols(built):
    lib = ctypes.CDLL(built)
    declared = _declared()
    assert declared, "no declarations found in include/"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_binding_lists_the_same_symbols(built):
    from qvb8_b200 import lib
    assert sorted(lib.EXPORTS) == _declared()
    assert b"sm_100a" in lib.load().qvb8_version()


def test_host_side_argument_checks_need_no_gpu(built):
    from qvb8_b200 import lib
    L = lib.load()
    assert L.qvb8_decode(None, 0, None, None) == 1                       # QVB8_ERR_ARG: null pack
    assert b"null pack" in L.qvb8_last_error()
    assert L.qvb8_small_m_scratch_bytes(0, 128, 128) == 0                # out-of-range sizes need no scratch


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from qvb8_b200 import lib
    monkeypatch.setattr(lib, "_lib", None)
    monkeypatch.setattr(lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or eager fallback"):
        lib.load()


def _describe(shapes, M, per_shape=1):
    """(list launches, list entries, single jobs) for products of the given (Q, P) shapes -- host arithmetic of the
    library, no device: the pointers only have to look aligned"""
    import ctypes
    from qvb8_b200 import lib
    L = lib.load()
    packs, jobs = [], (lib.JobStruct * (len(shapes) * per_shape))()
    k = 0
    for Q, P in shapes:
        for _ in range(per_shape):
            pk = lib.PackStruct()
            pk.ids, pk.ids_bytes, pk.min_s, pk.tau_s, pk.nbits, pk.bit_off = 0x10000, 1 << 30, 0x10000, 0x10000, 0x10000, 0x10000
            pk.Q, pk.P, pk.esc_idx, pk.esc_vals, pk.n_esc = Q, P, None, None, 0
            packs.append(pk)
            jobs[k].w = ctypes.pointer(pk)
            jobs[k].plan, jobs[k].X, jobs[k].Y = 0x20000, 0x30000, 0x40000
            jobs[k].x_dtype, jobs[k].x_mode = 1, 0
            k += 1
    a, b, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    rc = L.qvb8_small_m_group_describe(jobs, k, M, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
    assert rc == 0, L.qvb8_last_error()
    return a.value, b.value, c.value


def test_how_a_list_is_cut_into_launches(built):
    layer = [(6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288)]       # the four fused projections of a 9B layer
    # one token: nothing is cut; 128 jobs are one launch, 129 two
    assert _describe(layer, 1, per_shape=32) == (1, 128, 0)
    assert _describe(layer + [(512, 1024)], 1, per_shape=32)[:1] == (2,)
    # eight tokens: 12288 columns x 8 tokens = 192 KB of activations are cut into three column ranges (64 KB each), the
    # 4096-column products stay whole: 6 entries per layer
    assert _describe(layer, 8) == (1, 6, 0)
    assert _describe(layer, 8, per_shape=32) == (2, 192, 0)
    # four tokens: 96 KB -> two ranges
    assert _describe(layer, 4) == (1, 5, 0)
    # columns that are no multiple of 128 cannot stream: on their own
    assert _describe([(256, 4096), (256, 1000)], 1) == (0, 0, 2)            # (a list of one is a single launch too)
    assert _describe([(256, 4096), (256, 4096), (256, 1000)], 1) == (1, 2, 1)


def test_which_expert_layers_take_the_streaming_route(built):
    """host arithmetic: up to 8 tokens, column counts that are multiples of 128, at most 128 distinct experts"""
    import ctypes
    from qvb8_b200 import lib
    L = lib.load()

    def stack(Q, P, ids=0x10000):
        return lib.ExpertStackStruct(ids, 1 << 30, 0x10000, 0x10000, 0x10000, 0x10000, Q, P)

    def streams(M, topk, E, up, dn):
        return L.qvb8_moe_streams(M, topk, E, ctypes.byref(up), ctypes.byref(dn))
    up, dn = stack(1536, 2048), stack(2048, 768)                # the 35B-A3B-class expert: gate_up 1536 x 2048, down 2048 x 768
    assert [streams(M, 8, 128, up, dn) for M in (1, 4, 8, 9, 32)] == [1, 1, 1, 0, 0]
    assert streams(8, 8, 128, stack(192, 256), stack(256, 96)) == 0          # 96 columns: no multiple of 128
    assert streams(8, 8, 128, stack(1536, 2048, ids=0x10008), dn) == 0       # stack not 16-byte aligned
    assert streams(8, 32, 512, up, dn) == 0                                  # up to 256 distinct experts: too many jobs
    assert L.qvb8_moe_plan_bytes(128, 1536) > 128 * 102 * 400                # a plan per expert, a descriptor per tile
