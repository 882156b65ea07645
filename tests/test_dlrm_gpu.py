"""The recommendation model on the GPU: stage-by-stage bit-exactness against the CPU oracle,
end-to-end closeness, and partitioned == unpartitioned (the reference's own requirement,
tests/unittests/RecommendationSystemTest.cpp:1155-1226)."""
import numpy as np
import pytest
import torch

from glow_b200 import dlrm, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"

CFG = dict(tables=6, rows=3000, dim=32, batch=64, dense_in=48, bottom=(64, 32), top=(96, 48, 1), mean_len=12.0,
           max_len=40)


@pytest.fixture(scope="module", params=["symmetric", "asymmetric"])
def model(request):
    cfg = dlrm.DLRMConfig(**CFG, weights_schema=request.param)
    tables = {t: dlrm.make_table(cfg, t, DEV) for t in range(cfg.tables)}
    fm = dlrm.float_model(cfg)
    ranges = dlrm.calibrate(cfg, fm, tables, DEV)
    qm = dlrm.quantize_model(cfg, fm, ranges)
    return cfg, tables, fm, qm


def oracle_dense_part(oracle, cfg, qm, dense, pooled):
    """Quantize -> bottom MLP -> Dequantize -> interaction -> Quantize -> top MLP -> Dequantize."""
    x = oracle.element_quantize_i8(dense, *qm["dense_tqp"])
    for fc in qm["bottom"]:
        p = fc.params
        x = oracle.rowwise_quantized_fc_i8_i32(x, fc.w, fc.bias, fc.w_offsets, p[:3], p[3:], fc.out_offset, fc.in_offset, 0)
        if fc.relu:
            x = oracle.element_maxsplat_i8(x, fc.out_offset)
    last = qm["bottom"][-1]
    x0 = oracle.element_dequantize_i8(x, last.out_scale, last.out_offset)
    inter = oracle.pairwise_dot_interaction(x0, pooled)
    y = oracle.element_quantize_i8(inter, *qm["interaction_tqp"])
    for fc in qm["top"]:
        p = fc.params
        y = oracle.rowwise_quantized_fc_i8_i32(y, fc.w, fc.bias, fc.w_offsets, p[:3], p[3:], fc.out_offset, fc.in_offset, 0)
        if fc.relu:
            y = oracle.element_maxsplat_i8(y, fc.out_offset)
    last = qm["top"][-1]
    return y, oracle.element_dequantize_i8(y, last.out_scale, last.out_offset)


def test_single_gpu_against_oracle(oracle, model):
    cfg, tables, fm, qm = model
    rank = dlrm.DLRMRank(cfg, qm, tables, device=DEV)
    dense, lengths, indices = dlrm.make_request(cfg, 1, device=DEV)
    out = rank.forward_request(dense, lengths, indices).clone()
    torch.cuda.synchronize()
    assert int(rank.status.item()) == 0
    pooled_gpu = rank.slabs[0].cpu().numpy()
    # pooling stage: within the float tolerance of the strict CPU kernel
    for t in range(cfg.tables):
        n = int(lengths[t].sum())
        want = oracle.frwq_slws_u8_f32(tables[t].cpu().numpy(), np.ones(n, np.float32), indices[t].cpu().numpy(),
                                       lengths[t].cpu().numpy())
        np.testing.assert_allclose(pooled_gpu[:, t], want, rtol=1e-5, atol=1e-4)
    # everything after the pooled vectors: bit for bit
    q_want, f_want = oracle_dense_part(oracle, cfg, qm, dense.cpu().numpy(), pooled_gpu)
    np.testing.assert_array_equal(rank.act_t[-1].cpu().numpy(), q_want)
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), f_want.view(np.uint32))
    assert len(np.unique(q_want)) > 5
    # end to end against the fp32 model: quantisation error only (the reference accepts 0.005..0.02
    # of the output range against its Interpreter)
    pooled_t = torch.from_numpy(pooled_gpu).to(DEV)
    ref, _ = dlrm.float_forward(cfg, fm, dense, pooled_t)
    span = float(ref.max() - ref.min())
    assert float((out - ref).abs().max()) < 0.08 * span


@pytest.mark.parametrize("B,T,D", [(37, 9, 24), (19, 64, 128), (5, 6, 10), (3, 0, 8), (11, 15, 36)])
def test_interaction_kernel_bit_exact(oracle, B, T, D):
    """(D a multiple of 4: the register-tiled kernel; else the plain one; T = 0: no pairs at all)"""
    rng = np.random.default_rng(B + T + D)
    dense = rng.standard_normal((B, D)).astype(np.float32)
    pooled = rng.standard_normal((B, T, D)).astype(np.float32) * 3
    want = oracle.pairwise_dot_interaction(dense, pooled)
    got = ops.pairwise_dot_interaction(torch.from_numpy(dense).to(DEV), torch.from_numpy(pooled).to(DEV))
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # lower-triangle, row-major pair order
    v = np.concatenate([dense[:, None], pooled], 1).astype(np.float64)
    z = v @ v.transpose(0, 2, 1)
    ii, jj = np.tril_indices(T + 1, -1)
    if T:  # (an fp32 chain of D terms against float64: the pair ORDER is what this checks)
        np.testing.assert_allclose(want[:, D:], z[:, ii, jj], rtol=1e-4, atol=1e-4 * D)
    sc, off = 0.11, -7
    gq = ops.pairwise_dot_interaction(torch.from_numpy(dense).to(DEV), torch.from_numpy(pooled).to(DEV), quant=(sc, off))
    np.testing.assert_array_equal(gq.cpu().numpy(), oracle.element_quantize_i8(want, sc, off))


@pytest.mark.parametrize("world", [2, 3])
def test_partitioned_equals_unpartitioned(model, world):
    cfg, tables, fm, qm = model
    if cfg.batch % world:
        cfg = dlrm.DLRMConfig(**{**CFG, "batch": 66})
    whole = dlrm.DLRMRank(cfg, qm, tables, device=DEV)
    dense, lengths, indices = dlrm.make_request(cfg, 2, device=DEV)
    want = whole.forward_request(dense, lengths, indices).clone()
    ranks = [dlrm.DLRMRank(cfg, qm, {t: tables[t] for t in dlrm.tables_of_rank(cfg, r, world)}, r, world, DEV, "emulated")
             for r in range(world)]
    for r in ranks:
        r.set_peers(ranks)
    bound = [r.prepare({t: lengths[t] for t in r.my_tables}, {t: indices[t] for t in r.my_tables}, 0) for r in ranks]
    for r, b in zip(ranks, bound):  # every rank pools its tables for the whole batch ...
        r.pool_and_exchange(b, 0)
    outs = []
    for r in ranks:                 # ... then runs the dense layers on its slice
        lo, hi = dlrm.batch_slice(cfg, r.rank, world)
        outs.append(r.dense_forward(dense[lo:hi].contiguous(), r.slabs[0]).clone())
    torch.cuda.synchronize()
    assert torch.equal(torch.cat(outs), want)
    assert torch.equal(torch.cat([r.slabs[0] for r in ranks]), whole.slabs[0])


def test_peer_rendezvous_kernel_and_its_bounded_wait():
    """The flag rendezvous of the fused exchange on one GPU: a rank alone meets itself (twice:
    the step count advances), and a rank whose peer never signals gives up after its limit and
    says so through the status word -- the context stays usable."""
    buf = ops.PeerBuffer(8 * 3)
    flags = buf.as_tensor((24,), torch.uint8)
    flags.zero_()
    st = ops.new_status(DEV)
    alone = torch.tensor([buf.ptr], dtype=torch.int64, device=DEV)
    ops.peer_rendezvous(buf.ptr, alone, 1, 0, st)
    ops.peer_rendezvous(buf.ptr, alone, 1, 0, st)
    torch.cuda.synchronize()
    words = flags.view(torch.int64)
    assert int(st.item()) == 0 and int(words[0]) == 2 and int(words[1]) == 2
    # "two ranks", both mapped to this buffer, of which only rank 0 exists: slot 1 is never written
    flags.zero_()
    both = torch.tensor([buf.ptr, buf.ptr], dtype=torch.int64, device=DEV)
    ops.peer_rendezvous(buf.ptr, both, 2, 0, st, limit_cycles=2_000_000)  # about a millisecond
    torch.cuda.synchronize()
    assert int(st.item()) == 16
    st.zero_()
    ops.peer_rendezvous(buf.ptr, alone, 1, 0, st)  # and the next launch is fine
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    buf.release()
