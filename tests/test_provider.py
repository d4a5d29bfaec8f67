"""The backend provider (volvoxai_b200/provider/vxb200_provider.c) driven by a stand-in runtime.

libvxb200_provider.so is built against the reference's own public header
(native/include/volvoxai_backend.h); oracle/_ref/libvxfakehost.so (oracle/fake_host.c, built against
the same header) plays the runtime: it owns vx_backend_register_provider with the reference's
descriptor checks restated (native/src/runtime/backend_sdk.c:92-139) and drives runtime_create ->
compile -> context_create -> context_execute with HOST bindings and a copying output sink.
CPU part: the descriptor passes the exact-contract checks (struct size, ABI version, contract
marker and extent, name rules, required callbacks) and broken variants are rejected; on a box
without a B200 runtime_create reports BACKEND_UNAVAILABLE.  GPU part: the fixture packages compile
and execute through the provider with the reference's bytes.
"""
import ctypes as C
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
FAKE = os.path.join(ROOT, "oracle", "_ref", "libvxfakehost.so")
PROVIDER = os.path.join(ROOT, "volvoxai_b200", "libvxb200_provider.so")
PACKAGES = os.path.join(HERE, "golden", "packages")
OK, INVALID, UNAVAILABLE, UNSUPPORTED = 0, -1, -6, -7
DT_F32, DT_I8 = 18, 6
DYNAMIC_I8, F32_ARITH = 1, 3


@pytest.fixture(scope="module")
def host():
    if not (os.path.exists(FAKE) and os.path.exists(PROVIDER)):
        pytest.skip("provider or stand-in runtime not built (both need the reference's public header)")
    fake = C.CDLL(FAKE, mode=C.RTLD_GLOBAL)       # exports vx_backend_register_provider to the provider
    prov = C.CDLL(PROVIDER, mode=C.RTLD_GLOBAL)
    for name in ("fake_host_message", "fake_host_route_evidence", "fake_host_provider_name"):
        getattr(fake, name).restype = C.c_char_p
    fake.fake_host_contract_marker.restype = C.c_uint64
    fake.fake_host_provider_struct_size.restype = C.c_size_t
    fake.fake_host_max_rank.restype = C.c_size_t
    vp, sz = C.c_void_p, C.c_size_t
    fake.fake_host_compile.argtypes = [C.c_char_p, vp, sz, vp, vp, vp, vp, sz, sz, C.c_int, C.c_char_p]
    fake.fake_host_execute.argtypes = [vp, vp, vp, vp, vp, vp, sz, vp, vp, vp, vp, sz]
    fake.fake_host_register.argtypes = [vp]
    fake.fake_host_register_broken.argtypes = [vp, C.c_int]
    fake.fake_host_context_create.argtypes = [C.c_int]
    return fake, prov


def test_descriptor_passes_the_exact_contract_checks(host):
    fake, prov = host
    assert fake.fake_host_contract_marker() == 0x565850524F563032
    reg = C.cast(prov.vxb200_provider_register, C.c_void_p)
    assert fake.fake_host_register(reg) == OK
    assert fake.fake_host_provider_name() == b"b200-w8a8"
    assert fake.fake_host_register(reg) == INVALID      # duplicate name
    for variant in range(4):     # wrong struct size, wrong marker, reserved name, missing callback
        assert fake.fake_host_register_broken(C.cast(prov.vxb200_provider_descriptor, C.c_void_p), variant) == INVALID


def test_runtime_create_reports_unavailable_without_a_b200(host):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this box has a CUDA device")
    fake, prov = host
    fake.fake_host_register(C.cast(prov.vxb200_provider_register, C.c_void_p))
    assert fake.fake_host_runtime_create() == UNAVAILABLE
    assert fake.fake_host_message()


def specs(fake, entries):
    """entries: [(name, dtype, shape)] -> the flat arrays the stand-in runtime takes."""
    rank_cap = fake.fake_host_max_rank()
    names = (C.c_char_p * len(entries))(*[e[0].encode() for e in entries])
    dtypes = (C.c_uint32 * len(entries))(*[e[1] for e in entries])
    ranks = (C.c_uint32 * len(entries))(*[len(e[2]) for e in entries])
    dims = (C.c_int64 * (len(entries) * rank_cap))()
    for i, e in enumerate(entries):
        for a, d in enumerate(e[2]):
            dims[i * rank_cap + a] = d
    return names, dtypes, ranks, dims


def compile_package(fake, name, inputs, outputs, arithmetic=DYNAMIC_I8, policy=b"b200-w8a8"):
    folder = os.path.join(PACKAGES, name)
    weights = (C.c_char_p * 1)(os.path.join(folder, "model.safetensors").encode())
    names, dtypes, ranks, dims = specs(fake, inputs + outputs)
    return fake.fake_host_compile(os.path.join(folder, "graph.json").encode(), weights, 1, names, dtypes, ranks, dims,
                                  len(inputs), len(outputs), arithmetic, policy)


def execute(fake, inputs, arrays, outputs):
    names, dtypes, ranks, dims = specs(fake, inputs)
    data = (C.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
    nbytes = (C.c_size_t * len(arrays))(*[a.nbytes for a in arrays])
    outs = [np.zeros(shape, np.float32 if dt == DT_F32 else np.int8) for (_, dt, shape) in outputs]
    onames = (C.c_char_p * len(outs))(*[o[0].encode() for o in outputs])
    odt = (C.c_uint32 * len(outs))(*[o[1] for o in outputs])
    obuf = (C.c_void_p * len(outs))(*[o.ctypes.data for o in outs])
    obytes = (C.c_size_t * len(outs))(*[o.nbytes for o in outs])
    rc = fake.fake_host_execute(names, dtypes, ranks, dims, data, nbytes, len(arrays), onames, odt, obuf, obytes, len(outs))
    return rc, outs


@pytest.mark.gpu
def test_provider_compiles_and_executes_the_fixture_packages(host):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    fake, prov = host
    fake.fake_host_register(C.cast(prov.vxb200_provider_register, C.c_void_p))
    assert fake.fake_host_runtime_create() == OK
    # static W8A8 island
    ins, outs = [("x", DT_F32, (6, 96))], [("y", DT_F32, (6, 24)), ("y_q", DT_I8, (6, 24))]
    assert compile_package(fake, "static_island", ins, outs, policy=b"someone-else") == INVALID   # not in the policy
    assert compile_package(fake, "static_island", ins, [("y", DT_F32, (6, 25)), outs[1]]) == INVALID   # specs differ
    assert compile_package(fake, "static_island", ins, outs) == OK, fake.fake_host_message()
    assert fake.fake_host_route_attested() and b"provider=b200-w8a8" in fake.fake_host_route_evidence()
    assert fake.fake_host_context_create(1) == UNSUPPORTED          # decode-row contexts are not served
    assert fake.fake_host_context_create(0) == OK, fake.fake_host_message()
    want = np.load(os.path.join(PACKAGES, "static_island", "expected.npz"))
    rc, (y, y_q) = execute(fake, ins, [want["x"]], outs)
    assert rc == OK, fake.fake_host_message()
    assert np.array_equal(y_q, want["y_q"]) and np.array_equal(y.view(np.uint32), want["y"].view(np.uint32))
    assert b"fc1=static+" in fake.fake_host_route_evidence()
    rc, _ = execute(fake, [("x", DT_F32, (5, 96))], [want["x"][:5].copy()], outs)   # a binding of the wrong shape
    assert rc == INVALID
    fake.fake_host_teardown()
    # PackedLinear package written by the reference's exporter: attested for DYNAMIC_I8 only
    assert fake.fake_host_runtime_create() == OK
    ins, outs = [("x", DT_F32, (5, 96))], [("y", DT_F32, (5, 40))]
    assert compile_package(fake, "packed_w4", ins, outs, arithmetic=F32_ARITH) == UNSUPPORTED
    assert compile_package(fake, "packed_w4", ins, outs) == OK, fake.fake_host_message()
    assert fake.fake_host_context_create(0) == OK
    want = np.load(os.path.join(PACKAGES, "packed_w4", "expected.npz"))
    rc, (y,) = execute(fake, ins, [want["x"]], outs)
    assert rc == OK
    nan = np.isnan(want["y"])
    assert np.array_equal(np.isnan(y), nan) and np.array_equal(y[~nan].view(np.uint32), want["y"][~nan].view(np.uint32))
    fake.fake_host_teardown()
