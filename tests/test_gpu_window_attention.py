"""The tensor-core windowed attention kernel (csrc/attention_window.cu) against the general kernel on the same
pages, over sizes the model tests do not reach: key rows of odd multiples of 16, values narrower than keys, group
sizes that do not divide a block's rows, several requests of unequal lengths in one batch, steps of few rows (whose
key tiles are cut into runs and merged), pooled entries, slopes, a gate, value pages of their own."""

import pytest
import torch

from conftest import device

pytestmark = pytest.mark.gpu


def _case(seed, num_q, num_kv, dk, dv, v_own, window, pool, slopes, gate, q_lens, kv_lens, page=8):
    from ullm_b200.csrc import kernels
    from ullm_b200.engine.batch import Workspace

    K = kernels()
    dev = device()
    g = torch.Generator().manual_seed(seed)
    R, T = len(q_lens), sum(q_lens)
    max_pages = max(-(-n // page) for n in kv_lens) + 1
    pages = R * max_pages + 3
    perm = torch.randperm(pages, generator=g).tolist()  # a request's pages lie anywhere
    bt = torch.full((R + 2, max_pages), -1, dtype=torch.int32)
    slots = [R + 1 - r if r < 2 else r for r in range(R)]  # batch row r reads another row of the table
    for r in range(R):
        for i in range(-(-kv_lens[r] // page)):
            bt[slots[r], i] = perm.pop()
    bf = torch.bfloat16
    k_pages = (torch.randn(pages, page, num_kv, dk, generator=g) * 0.7).to(bf).to(dev)
    v_pages = (torch.randn(pages, page, num_kv, dv, generator=g)).to(bf).to(dev) if v_own else None
    pooled = None
    if pool:
        p_max = max(1, -(-(max(kv_lens) // pool) // page))
        p_pages = R * p_max + 2
        pperm = torch.randperm(p_pages, generator=g).tolist()
        pbt = torch.full((R + 2, p_max), -1, dtype=torch.int32)
        for r in range(R):
            for i in range(-(-(kv_lens[r] // pool) // page)):
                pbt[slots[r], i] = pperm.pop()
        pk = (torch.randn(p_pages, page, num_kv, dk, generator=g) * 0.7).to(bf).to(dev)
        pv = torch.randn(p_pages, page, num_kv, dv, generator=g).to(bf).to(dev) if v_own else None
        pooled = (pk, pv, pbt.to(dev))
    extra = 16  # q rows are a column range of wider rows
    q = (torch.randn(T, num_q * dk + extra, generator=g)).to(bf).to(dev)
    gate_t = torch.randn(T, num_q * dv, generator=g).to(bf).to(dev) if gate else None
    sl = None
    if slopes:
        sl = (2.0 ** (-8.0 * torch.arange(1, num_q + 1) / num_q)).float().to(dev)
    cu = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device=dev)
    tr = torch.tensor([r for r, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32, device=dev)
    rs = torch.tensor(slots, dtype=torch.int32, device=dev)
    ws = Workspace(dev, max_tokens=T, max_requests=R)
    outs = {}
    for tc in (False, True):
        old = K.window_attention_tc
        K.window_attention_tc = tc
        try:
            out = torch.full((T, num_q * dv + 8), 7.0, dtype=bf, device=dev)  # (a column range of wider rows)
            K.windowed_attention(q[:, :num_q * dk], out[:, :num_q * dv], k_pages, v_pages, bt.to(dev), rs, cu, kvl, tr,
                                 num_q, num_kv, dk, dv, page, window, dk ** -0.5, slopes=sl, pool=pool, pooled=pooled,
                                 gate=gate_t, out_scale=0.75, num_requests=R, workspace=ws)
            torch.cuda.synchronize()
            K.raise_on_status()
            assert K.attention_path == ("window_mma" if tc else "generic"), K.attention_path
            assert (out[:, num_q * dv:] == 7.0).all(), "columns beside the output were written"
            outs[tc] = out[:, :num_q * dv].float().cpu()
        finally:
            K.window_attention_tc = old
    ref, got = outs[False], outs[True]
    assert torch.isfinite(got).all()
    scale = float(ref.abs().max())
    err = float((got - ref).abs().max()) / scale
    rms = float((got - ref).pow(2).mean().sqrt()) / scale
    assert err <= 2.5e-2 and rms <= 3e-3, f"max err {err:.2e}, rms {rms:.2e} of scale"


CASES = [
    # num_q, num_kv, dk, dv, value pages, window, pool, slopes, gate, q lengths, kv lengths
    (6, 2, 80, 80, False, 37, 0, False, False, [70, 3, 1], [70, 50, 131]),
    (5, 1, 48, 32, False, 20, 5, False, False, [1, 1, 1], [97, 20, 203]),       # few rows: runs + merge, pooled
    (7, 7, 16, 16, True, 0, 0, True, True, [33, 2], [40, 2]),                    # no window
    (12, 4, 96, 96, True, 70, 0, True, True, [130, 1, 9], [130, 300, 77]),
    (3, 1, 208, 176, False, 65, 0, False, False, [20, 45], [150, 45]),           # two column groups, 13 steps
    (2, 1, 336, 320, False, 129, 16, False, False, [1, 90], [400, 260]),         # three column groups, pooled
    (4, 1, 448, 384, False, 100, 0, False, False, [1, 1], [257, 64]),            # constant-size instance, runs
    (8, 2, 128, 128, True, 64, 64, False, False, [64, 64, 1], [64, 192, 513]),   # window = pool = a tile
    (16, 2, 64, 64, False, 1, 1, False, True, [5, 1], [5, 66]),                  # window of one, blocks of one
    (64, 1, 32, 32, False, 9, 2, False, False, [3, 1], [30, 11]),                # a token's heads fill a block
]


@pytest.mark.parametrize("case", range(len(CASES)))
def test_tensor_core_kernel_against_the_general_kernel(case):
    _case(100 + case, *CASES[case])
