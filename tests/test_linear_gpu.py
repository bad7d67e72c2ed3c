"""``QVBandLinearV8.forward`` on the GPU: every route of ``choose_route`` against the CPU oracle, plain and
bf16-certified packs, bias, dtype handling, row subsets.  Plus the route table itself (CPU)."""
import numpy as np
import pytest
import torch

import oracle
from qvb8_b200 import linear, synth
from qvb8_b200.linear import QVBandLinearV8, Route, choose_route
from util import pack_np, rel_fro

DEV = "cuda:0"
TOL = 1e-2


def test_route_table():
    bf, h = torch.bfloat16, torch.float16
    assert choose_route(1, bf, True, True, 4096) == Route("stream", 1, "fp16", 0)      # fewer than 8 rows: fp16 table
    assert choose_route(7, bf, True, False, 4096) == Route("stream", 1, "fp16", 0)
    assert choose_route(8, bf, True, False, 4096) == Route("stream", 1, "bf16", 1)     # bf16 mode from 8 rows on
    assert choose_route(48, bf, False, False, 4096) == Route("stream", 1, "fp16", 0)
    assert choose_route(49, h, True, False, 4096) == Route("stream", 2, "fp16", 0)
    assert choose_route(96, bf, True, False, 4096) == Route("stream", 2, "bf16", 1)
    assert choose_route(97, bf, True, True, 4096) == Route("dense", 0, "bf16", 1)
    assert choose_route(97, bf, True, False, 4096).kind in ("dense", "fused")
    assert choose_route(300, h, False, False, 100).kind == "dense"


@pytest.mark.gpu
@pytest.mark.parametrize("restore", ["fp16", "fp16+bf16"])
@pytest.mark.parametrize("M", [1, 8, 48, 97, 300])
def test_forward_against_the_oracle(cuda_lib, restore, M):
    Q, P = 320, 1024
    pk = synth.synth_pack(Q, P, seed=17, tau=2e-3, device=DEV, restore=restore)
    bias = torch.linspace(-0.5, 0.5, Q, device=DEV)
    lin = QVBandLinearV8.from_pack(pk, bias=bias)
    d = pack_np(pk)
    for xdt in (torch.bfloat16, torch.float16, torch.float32):
        X = synth.synth_activation(M, P, seed=M, device=DEV, dtype=xdt)
        route = lin.route_for(M, xdt)
        y = lin(X.reshape(1, M, P))
        assert y.shape == (1, M, Q) and y.dtype == xdt
        W = oracle.qvb8_dense(d, table=route.table)
        want = oracle.matmul_f32w(X.float().cpu().numpy(), W, narrow_x=route.x_mode == 0) + bias.cpu().numpy()[None, :]
        err = rel_fro(y.float().cpu().numpy().reshape(M, Q), want)
        # fp32 activations give an fp32 result (fp16-rounded weights on the dense route: 5e-4); 16-bit results carry
        # their own output rounding (bf16: 4e-3)
        assert err < (1e-3 if xdt == torch.float32 else TOL), (xdt, route, err)


@pytest.mark.gpu
def test_bf16_gemm_route_and_restores(cuda_lib):
    Q, P = 192, 512
    pk = synth.synth_pack(Q, P, seed=23, tau=2e-3, device=DEV, restore="fp16+bf16")
    lin = QVBandLinearV8.from_pack(pk)
    assert linear.enable_bf16_gemm(torch.nn.Sequential(lin)) == (1, 1)
    X = synth.synth_activation(200, P, seed=2, device=DEV, dtype=torch.bfloat16)
    assert lin.route_for(200, X.dtype) == Route("dense", 0, "bf16", 1)
    y = lin(X)
    d = pack_np(pk)
    Wb = oracle.decode_16(d["ids"], d["nbits"], d["bit_off"], d["min_s"], d["tau_s"], Q, P, d["esc_idx_bf16"],
                          d["esc_vals_bf16"], "bf16")
    assert np.array_equal(lin.dense(torch.bfloat16).cpu().view(torch.int16).numpy().view(np.uint16), Wb)
    W = torch.from_numpy(Wb.view(np.int16)).view(torch.bfloat16).float().numpy()
    want = oracle.matmul_f32w(X.float().cpu().numpy(), W, narrow_x=False)
    assert rel_fro(y.float().cpu().numpy(), want) < TOL
    rep = linear.footprint_report(lin)
    assert rep["linears"] == 1 and rep["params"] == Q * P and 0.5 < rep["bytes_per_param"] < 1.2


@pytest.mark.gpu
def test_row_subset_module_on_the_device(cuda_lib):
    pk = synth.synth_pack(256, 512, seed=5, device=DEV)
    lin = QVBandLinearV8.from_pack(pk)
    rows = torch.tensor([200, 3, 77, 78, 255, 0, 128] + list(range(16, 48)), device=DEV)
    sub = lin.row_subset(rows)
    assert sub.ids.data_ptr() == lin.ids.data_ptr()                    # no payload bytes copied
    X = synth.synth_activation(3, 512, seed=1, device=DEV)
    assert torch.equal(sub(X), lin(X)[:, rows])
    assert torch.equal(sub.dense(torch.float16), lin.dense(torch.float16)[rows])


@pytest.mark.gpu
def test_casts_keep_the_fp32_metadata_and_graph_capture_works(cuda_lib):
    pk = synth.synth_pack(128, 4096, seed=6, device=DEV)
    lin = QVBandLinearV8.from_pack(pk).to(torch.bfloat16)
    assert lin.min_s.dtype == torch.float32 and lin.esc_vals.dtype == torch.float32
    X = synth.synth_activation(4, 4096, seed=1, device=DEV)
    want = lin(X)
    lin.reserve(8)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        lin.reserve(8)                                                 # scratch is kept per stream
        y = lin(X)
    s.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        y = lin(X)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, want)
