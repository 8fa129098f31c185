"""Peer-memory byte exchange of the staged pipeline, every rank emulated on one GPU, against plain indexing."""
import pytest
import torch

from coccl_b200.ops import exchange as X

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,frames,stride", [(2, 1, 4096), (4, 1, 1 << 20), (4, 3, 48 * 1024 + 16), (8, 2, 1 << 18)])
@pytest.mark.parametrize("gather", [False, True])
def test_exchange_of_full_blocks(cuda, n, frames, stride, gather):
    torch.manual_seed(n * 7 + frames)
    block = frames * stride
    send = [torch.randint(0, 256, ((1 if gather else n) * block,), dtype=torch.uint8, device=cuda) for _ in range(n)]
    state = {}
    for epoch in (1, 2):   # flags and staging are reused
        recv, _, state = X.emulate(send, gather=gather, frames=frames, frame_stride=stride, state=state, epoch=epoch,
                                   max_ctas=max(1, 296 // n))
        torch.cuda.synchronize()
        X.check_state(state)
        for d in range(n):
            for s in range(n):
                want = send[s] if gather else send[s][d * block:(d + 1) * block]
                assert torch.equal(recv[d][s * block:(s + 1) * block], want), (epoch, d, s)
        send = [t.flip(0).contiguous() for t in send]


@pytest.mark.parametrize("gather", [False, True])
def test_exchange_of_frames_moves_only_what_exists(cuda, gather):
    """Variable-size frames: the size comes from the device-side metadata; bytes behind it are not moved (the receive
    buffer keeps its zeros there), the records arrive in source order, raw and empty frames included."""
    n, frames, stride = 4, 5, 96 * 1024
    torch.manual_seed(3)
    blocks = 1 if gather else n
    send = [torch.randint(1, 256, (blocks * frames * stride,), dtype=torch.uint8, device=cuda) for _ in range(n)]
    meta = []
    for r in range(n):
        sizes = torch.randint(0, stride + 1, (blocks * frames,), device=cuda)
        sizes[0] = stride            # a full (raw) frame
        sizes[-1] = 0                # an empty one
        sizes[1] = 17                # not a multiple of 16: whole vectors travel, the record keeps the exact size
        enc = torch.randint(0, 2, (blocks * frames,), device=cuda)
        meta.append(torch.stack([sizes, enc], dim=1).to(torch.int64).contiguous())
    recv, rmeta, state = X.emulate(send, gather=gather, frames=frames, frame_stride=stride, meta=meta)
    torch.cuda.synchronize()
    X.check_state(state)
    for d in range(n):
        for s in range(n):
            for f in range(frames):
                src_frame = (0 if gather else d) * frames + f
                size = int(meta[s][src_frame, 0].item())
                got = recv[d][(s * frames + f) * stride:(s * frames + f + 1) * stride]
                want = send[s][src_frame * stride:(src_frame + 1) * stride]
                assert torch.equal(got[:size], want[:size]), (d, s, f)
                moved = (size + 15) // 16 * 16
                assert int(got[moved:].max().item()) == 0 if moved < stride else True
                assert torch.equal(rmeta[d][s * frames + f], meta[s][src_frame])


def test_exchange_wait_runs_out_when_a_peer_never_stores(cuda):
    """A flag that nothing sets: rank 0 runs alone in the production form, its stores go to a sink standing in for
    rank 1, and nobody stores into ITS inbox. With a 50 ms limit the wait gives up, the status word names phase and
    peer, and the context stays usable; nothing hangs or traps."""
    n, stride = 2, 4096
    send = [torch.zeros(n * stride, dtype=torch.uint8, device=cuda) for _ in range(n)]
    _, _, state = X.emulate(send, gather=False, frames=1, frame_stride=stride, epoch=5)
    torch.cuda.synchronize()
    X.check_state(state)
    state["flags"][0].zero_()
    import coccl_b200._lib as L
    import ctypes as C
    a = L.ExchangeArgs()
    pieces, pb = X.pieces_for(1, stride)
    a.nRanks, a.rankBase, a.gather, a.frames, a.pieces, a.frameStride, a.pieceBytes = 2, 0, 0, 1, pieces, stride, pb
    a.epoch, a.timeoutNs = 9, int(50e6)
    recv = torch.zeros(n * stride, dtype=torch.uint8, device=cuda)
    sink = torch.zeros(X.staging_bytes(2, 1, stride), dtype=torch.uint8, device=cuda)
    sink_flags = torch.zeros_like(state["flags"][0])
    a.send[0], a.recv[0] = send[0].data_ptr(), recv.data_ptr()
    # rank 0 alone (production form): its stores go to a sink standing in for rank 1, nobody stores into ITS inbox
    a.staging[0], a.flags[0], a.status[0] = state["staging"][0].data_ptr(), state["flags"][0].data_ptr(), state["status"][0].data_ptr()
    a.staging[1], a.flags[1], a.status[1] = sink.data_ptr(), sink_flags.data_ptr(), state["status"][1].data_ptr()
    fn = L.declare("cocclkPeerExchange", C.c_int, [C.POINTER(L.ExchangeArgs), C.c_int, C.c_int, C.c_void_p])
    assert fn(C.byref(a), 1, 4, L.cur_stream()) == 0
    torch.cuda.synchronize()
    code = int(state["status"][0][0].item()) & 0xFFFFFFFF
    assert code & 0x80000000 and ((code >> 23) & 0xff) == 6 and ((code >> 15) & 0xff) == 1   # phase 6, peer 1
