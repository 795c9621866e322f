"""The tensor-parallel exchange (eb_comm_*, eb_allreduce, the exchange inside eb_gemm_allreduce and
eb_decode_chain) on ONE GPU.

Ranks of a real group are separate processes on separate GPUs (tests/test_tp_gpu.py, and the
`--check` mode of bench.py).  Here the other rank is played by the test itself: before the
launch it writes the lines that rank would send, carrying the sequence number the kernel will
expect, into this rank's receive area; after the launch it reads what the kernel sent to the
"peer" area.  Nothing waits on another kernel, so nothing can hang; a wait that nobody satisfies
is exercised with a budget of a few milliseconds and must end in EB_ETIMEDOUT."""
import numpy as np
import pytest
import torch

from test_gemm_gpu import reference, check_close, status_ok

pytestmark = pytest.mark.gpu

LINES = 8 << 20                      # flagged-line region of the test contexts
SIGNALS = 4096                       # signal words in front of it (csrc/comm.cuh)


def make_ctx(world=2, budget=None, bulk=0):
    """Rank 0 of `world` over two local buffers: its own receive area and one that stands for
    every peer's.  Area = signal words | flagged-line region | bulk region."""
    from energonai_b200.comm import PeerExchange
    mine = torch.zeros(SIGNALS + LINES + bulk, dtype=torch.uint8, device="cuda")
    peer = torch.zeros(SIGNALS + LINES + bulk, dtype=torch.uint8, device="cuda")
    ctx = PeerExchange.from_pointers(0, world, mine, [mine.data_ptr()] + [peer.data_ptr()] * (world - 1), line_bytes=LINES,
                                     wait_budget_s=budget)
    return ctx, mine, peer


def pack_lines(values16, seq):
    """values16: uint16 numpy array (a multiple of 4 values) -> uint32 array of flagged lines
    {payload0, seq, payload1, seq} (the layout described in csrc/comm.cuh)."""
    pay = values16.reshape(-1, 2, 2).copy().view(np.uint32).reshape(-1, 2)
    out = np.empty((pay.shape[0], 4), dtype=np.uint32)
    out[:, 0], out[:, 2] = pay[:, 0], pay[:, 1]
    out[:, 1] = out[:, 3] = seq
    return out.reshape(-1)


def write_lines(area, half, first_line, lines_u32):
    off = SIGNALS + half * (LINES // 2) + first_line * 16
    area[off:off + lines_u32.size * 4] = torch.from_numpy(lines_u32.view(np.uint8)).cuda()


def read_payload16(area, half, first_line, n_lines):
    off = SIGNALS + half * (LINES // 2) + first_line * 16
    raw = area[off:off + n_lines * 16].cpu().numpy().view(np.uint32).reshape(-1, 4)
    return raw[:, [0, 2]].copy().view(np.uint16).reshape(-1), raw[:, 1], raw[:, 3]


def as_u16(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16).reshape(-1)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_allreduce_single_rank_is_identity_and_advances(dtype):
    from energonai_b200.comm import PeerExchange
    area = torch.zeros(SIGNALS + LINES, dtype=torch.uint8, device="cuda")
    ctx = PeerExchange.from_pointers(0, 1, area, [area.data_ptr()])
    x = torch.randn(3000, device="cuda").to(dtype)
    want = x.clone()
    for _ in range(3):                       # consecutive exchanges alternate the halves
        ctx.all_reduce(x)
    torch.cuda.synchronize()
    assert torch.equal(x, want) and ctx.status()[0] == 0
    ctx.destroy()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_allreduce_adds_the_peer_contribution(dtype):
    ctx, mine, peer = make_ctx()
    n = 4096
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(n, device="cuda", generator=g).to(dtype)
    other = torch.randn(n, device="cuda", generator=g).to(dtype)
    for seq in (1, 2):                       # two exchanges: halves 1, 0
        x0 = x.clone()
        write_lines(mine, seq & 1, 1 * (n // 4), pack_lines(as_u16(other), seq))       # source 1's slot
        ctx.all_reduce(x)
        torch.cuda.synchronize()
        assert ctx.status()[0] == 0
        assert torch.equal(x, (x0.float() + other.float()).to(dtype))
        sent, f0, f1 = read_payload16(peer, seq & 1, 0, n // 4)                         # what rank 0 sent: slot 0
        assert np.array_equal(sent, as_u16(x0)) and (f0 == seq).all() and (f1 == seq).all()
    ctx.destroy()


def test_allreduce_gives_up_when_the_peer_never_writes():
    """A flag that nothing sets: the wait runs out after its budget, the call returns, the
    context reports EB_ETIMEDOUT and the device stays usable."""
    ctx, mine, peer = make_ctx(budget=0.005)
    x = torch.ones(1024, device="cuda", dtype=torch.float16)
    ctx.all_reduce(x)
    torch.cuda.synchronize()
    code, where, _, detail = ctx.status()
    assert code == -4 and where == 20 and detail == 1
    assert ctx.status()[0] == 0              # cleared by the read above
    y = torch.ones(8, device="cuda") * 2
    assert float(y.sum()) == 16.0
    ctx.destroy()


def test_limits_are_refused():
    ctx, mine, peer = make_ctx()
    big = torch.zeros(LINES, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="receive area"):
        ctx.all_reduce(big)
    with pytest.raises(RuntimeError, match="8"):
        ctx.all_reduce(torch.zeros(3, device="cuda", dtype=torch.float16))
    ctx.destroy()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(16, 512, 1024), (3, 2048, 256), (16, 5120, 640), (40, 640, 4096), (128, 256, 512)])
def test_gemm_allreduce_with_host_written_peer(M, N, K, dtype):
    """eb_gemm_allreduce as rank 0 of 2: result = own product + the peer's lines + bias + residual,
    and the lines it sent carry its own product.  Receive layout of this kernel:
    [source][output column n][BN / 4 lines], BN = batch padded to 16 / 32 / 64 / 128."""
    from energonai_b200.gemm import gemm
    ctx, mine, peer = make_ctx()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(dtype)
    bias = torch.randn(N, device="cuda", generator=g).to(dtype)
    res = torch.randn(M, N, device="cuda", generator=g).to(dtype)
    other = (torch.randn(M, N, device="cuda", generator=g) * 2).to(dtype)          # the peer's partial product
    BN = ctx._padded(M)
    for seq in (1, 2, 3):
        padded = torch.zeros(N, BN, device="cuda", dtype=dtype)
        padded[:, :M] = other.t()
        write_lines(mine, seq & 1, 1 * N * (BN // 4), pack_lines(as_u16(padded), seq))
        out = gemm(a, w, bias=bias, residual=res, peer=ctx)
        torch.cuda.synchronize()
        status_ok()
        own = (a.float() @ w.float().t()).to(dtype)                                 # travels rounded to the operand type
        sent, f0, _ = read_payload16(peer, seq & 1, 0, N * (BN // 4))
        sent = torch.from_numpy(sent.view(np.int16).reshape(N, BN)[:, :M].copy()).cuda().view(dtype).t()
        assert (f0 == seq).all()
        check_close(sent, a.float() @ w.float().t(), dtype)
        want = sent.float() + other.float() + bias.float() + res.float()
        check_close(out, want, dtype)            # `sent` is what really travelled: one rounding left
    ctx.destroy()


def close_after_exchange(out, ref, part, dtype):
    """An exchanged product is rounded to the operand type before it travels and the sum is
    rounded again: two roundings, the first at the magnitude of the partial product `part`
    (whose last bit also depends on the order the fp32 partial sums were added in)."""
    from test_gemm_gpu import REL
    err = (out.float() - ref).abs()
    bound = REL[dtype] * (ref.abs() + 2 * part.abs()) + 4e-4 * ref.abs().max().clamp_min(1e-3)
    bad = err > bound
    assert not bad.any(), f"max err {err.max().item():.4g} at {int(bad.sum())} elements (ref max {ref.abs().max().item():.4g})"


def layer_tail(g, M, h, f, v, dtype):
    rnd = lambda *s, scale=1.0: (torch.randn(*s, device="cuda", generator=g) * scale).to(dtype)
    return dict(ctx=rnd(M, h), x=rnd(M, h), wo=rnd(h, h, scale=0.03), bo=rnd(h, scale=0.1), g2=1 + rnd(h, scale=0.1),
                b2=rnd(h, scale=0.1), w1=rnd(f, h, scale=0.03), b1=rnd(f, scale=0.1), w2=rnd(h, f, scale=0.03),
                bb2=rnd(h, scale=0.1), g3=1 + rnd(h, scale=0.1), b3=rnd(h, scale=0.1), wv=rnd(v, h, scale=0.03),
                p1=rnd(M, h, scale=0.5), p2=rnd(M, h, scale=0.5))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("world", [1, 2])
@pytest.mark.parametrize("M,h,f,v", [(16, 256, 1024, 520), (16, 5120, 2560, 1923), (5, 1024, 4096, 6284), (100, 768, 3072, 2304)])
def test_chain_with_exchanged_products(M, h, f, v, world, dtype):
    """The tail of a tensor-parallel decoder layer in one launch:
    out-proj (exchanged) -> sum + bias + residual + LayerNorm -> FC1 -> FC2 (exchanged) ->
    sum + bias + residual + LayerNorm -> projection.  world 1: the rank exchanges with itself.
    world 2: the peer's two contributions (p1, p2) are written by the test beforehand.  Receive
    layout of the chain: [source][batch row m][N / 4 lines]."""
    from energonai_b200.chain import Chain, gemm_op, reduce_layernorm_op
    from energonai_b200.comm import PeerExchange
    eps = 1e-5
    g = torch.Generator(device="cuda").manual_seed(M * 3 + h + world)
    t = layer_tail(g, M, h, f, v, dtype)
    if world == 1:
        area = torch.zeros(SIGNALS + LINES, dtype=torch.uint8, device="cuda")
        ctx = PeerExchange.from_pointers(0, 1, area, [area.data_ptr()])
        mine = area
    else:
        ctx, mine, peer = make_ctx()
    new = lambda *s, dt=dtype: torch.full(s, float("nan"), device="cuda", dtype=dt)
    x1, n, a, x2, y = new(M, h), new(M, h), new(M, f), new(M, h), new(M, v, dt=torch.float32)
    ops = [gemm_op(t["ctx"], t["wo"], exchange=True),
           reduce_layernorm_op(x1, h, bias=t["bo"], residual=t["x"], y=n, gamma=t["g2"], beta=t["b2"], eps=eps),
           gemm_op(n, t["w1"], a, bias=t["b1"], act="relu"),
           gemm_op(a, t["w2"], exchange=True),
           reduce_layernorm_op(x2, h, bias=t["bb2"], residual=x1, y=n, gamma=t["g3"], beta=t["b3"], eps=eps),
           gemm_op(n, t["wv"], y)]
    ch = Chain(ops, M, dtype, "cuda", comm=ctx)
    first = None
    for launch in range(3):
        seq1, seq2 = 2 * launch + 1, 2 * launch + 2
        if world == 2:
            write_lines(mine, seq1 & 1, 1 * M * (h // 4), pack_lines(as_u16(t["p1"]), seq1))
            write_lines(mine, seq2 & 1, 1 * M * (h // 4), pack_lines(as_u16(t["p2"]), seq2))
        ch.run()
        torch.cuda.synchronize()
        status_ok()
        p1 = t["p1"].float() if world == 2 else 0.0
        p2 = t["p2"].float() if world == 2 else 0.0
        own1 = (t["ctx"].float() @ t["wo"].float().t()).to(dtype).float()
        close_after_exchange(x1, own1 + p1 + t["bo"].float() + t["x"].float(), own1, dtype)
        ln2 = torch.nn.functional.layer_norm(x1.float(), (h,), t["g2"].float(), t["b2"].float(), eps)
        # (the chain's own normalised row is overwritten by the second LayerNorm: FC1 is compared
        # against a recomputed one, relative to the row maximum, a few output roundings)
        want_a = reference(ln2.to(dtype), t["w1"], t["b1"], "relu")
        tol = {torch.float16: 4e-3, torch.bfloat16: 3e-2}[dtype]
        assert ((a.float() - want_a).abs().amax(-1) <= tol * want_a.abs().amax(-1).clamp_min(1e-3)).all()
        own2 = (a.float() @ t["w2"].float().t()).to(dtype).float()
        close_after_exchange(x2, own2 + p2 + t["bb2"].float() + x1.float(), own2, dtype)
        ln3 = torch.nn.functional.layer_norm(x2.float(), (h,), t["g3"].float(), t["b3"].float(), eps)
        check_close(n, ln3, dtype)
        check_close(y, reference(n, t["wv"]), torch.float32)
        if first is None:
            first = y.clone()
        else:
            assert torch.equal(y, first)        # launches are reproducible bit for bit
    ctx.destroy()


def test_chain_exchange_gives_up_when_the_peer_never_writes():
    from energonai_b200.chain import Chain, gemm_op, reduce_layernorm_op
    from energonai_b200.gemm import device_status
    ctx, mine, peer = make_ctx(budget=0.005)
    M, h = 16, 256
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g).half()
    x1, n = torch.zeros(M, h, device="cuda").half(), torch.zeros(M, h, device="cuda").half()
    ops = [gemm_op(rnd(M, h), rnd(h, h), exchange=True),
           reduce_layernorm_op(x1, h, residual=rnd(M, h), y=n, gamma=rnd(h), beta=rnd(h))]
    Chain(ops, M, torch.float16, "cuda", comm=ctx).run()
    torch.cuda.synchronize()
    code, where, _, _ = device_status()
    assert code == -4 and where == 10
    assert device_status()[0] == 0
    ctx.destroy()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("world", [1, 2])
@pytest.mark.parametrize("M,N,K", [(256, 512, 128), (1000, 1024, 640), (2048, 5120, 640), (300, 264, 2560)])
def test_prompt_sized_row_parallel_sum(M, N, K, world, dtype):
    """eb_gemm_reduce_scatter + eb_reduce_broadcast as rank 0.  world 1: the whole sum lands in the
    gather area.  world 2: the test plays rank 1: it writes rank 1's partial of rank 0's rows into
    rank 0's staging area and pre-sets the two barrier words; afterwards rank 0's rows of the
    gather areas of BOTH ranks hold own + peer + bias + residual, and the tiles of the rows rank 1
    owns have arrived in rank 1's staging area.  Staging layout: [source][row in block][N]; rows
    are dealt out in blocks of whole 128-row tiles."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K + world)
    a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(dtype)
    bias = torch.randn(N, device="cuda", generator=g).to(dtype)
    res = torch.randn(M, N, device="cuda", generator=g).to(dtype)
    rpr = -(-(-(-M // 128)) // world) * 128                  # rows per rank: whole 128-row tiles
    bulk = (3 * max(world * rpr, M) * N * 2 + 4096) // 512 * 512
    own = (a.float() @ w.float().t())
    if world == 1:
        from energonai_b200.comm import PeerExchange
        area = torch.zeros(SIGNALS + LINES + bulk, dtype=torch.uint8, device="cuda")
        ctx = PeerExchange.from_pointers(0, 1, area, [area.data_ptr()], line_bytes=LINES)
        for _ in range(3):                                    # gather areas alternate, barrier numbers advance
            out = ctx.row_parallel(a, w, bias=bias, residual=res)
            torch.cuda.synchronize()
            assert ctx.status()[0] == 0
            close_after_exchange(out, own.to(dtype).float() + bias.float() + res.float(), own, dtype)
        ctx.destroy()
        return
    ctx, mine, peer = make_ctx(bulk=bulk)
    other = (torch.randn(rpr, N, device="cuda", generator=g) * 2).to(dtype)       # rank 1's partial of rank 0's rows
    stage_b = (world * rpr * N * 2 + 511) // 512 * 512
    gather_b = (M * N * 2 + 511) // 512 * 512
    B0 = SIGNALS + LINES                                                         # start of the bulk region
    for call in (1, 2):
        mine[B0 + rpr * N * 2: B0 + 2 * rpr * N * 2] = other.view(torch.uint8).view(-1)     # staging slot of source 1
        sig = mine[:64].view(torch.int32)
        sig[1] = call                                                             # slot 0 (start barrier), source 1
        sig[8 + 1] = call                                                         # slot 1 (end barrier), source 1
        out = ctx.row_parallel(a, w, bias=bias, residual=res)
        torch.cuda.synchronize()
        assert ctx.status()[0] == 0
        mine_rows = min(rpr, M)
        want = own[:mine_rows].to(dtype).float() + other[:mine_rows].float() + bias.float() + res[:mine_rows].float()
        close_after_exchange(out[:mine_rows], want, own[:mine_rows], dtype)
        goff = B0 + stage_b + (call - 1) * gather_b
        sent = peer[goff: goff + mine_rows * N * 2].view(dtype).view(mine_rows, N)
        assert torch.equal(sent, out[:mine_rows])                                 # the same rows went to the peer
        if M > rpr:                                                               # tiles of the peer's rows, in ITS staging slot 0
            theirs = peer[B0: B0 + (M - rpr) * N * 2].view(dtype).view(M - rpr, N)
            from test_gemm_gpu import check_close
            check_close(theirs, own[rpr:], dtype)
        psig = peer[:64].view(torch.int32)
        assert int(psig[0]) == call and int(psig[8]) == call                      # rank 0 announced itself at both barriers
    ctx.destroy()


def test_bulk_barrier_gives_up_when_the_peer_never_arrives():
    ctx, mine, peer = make_ctx(budget=0.005, bulk=8 << 20)
    a = torch.randn(256, 128, device="cuda").half()
    w = torch.randn(256, 128, device="cuda").half()
    ctx.row_parallel(a, w)
    torch.cuda.synchronize()
    code, where, _, detail = ctx.status()
    assert code == -4 and where in (21, 22) and detail == 1
    ctx.destroy()
