"""The multi-GPU output exchange on ONE GPU: two pools play rank 0 and rank 1 with every receive
buffer in this GPU's own memory, stepped one after the other on one stream (no kernel ever
waits for a kernel that has not been launched before it).  Same kernels as the multi-GPU path: the
combine kernel's flagged-word stores, the parity buffers and the bounded receiving kernel."""

import pytest
import torch

from helpers import make_case, pool_from_case

pytestmark = pytest.mark.gpu


def _two_ranks(wait_polls=0):
    from pqhsa_release_b200.parallel import LocalPeerGroup

    cases = [make_case(B=2, Hkv=1, G=4, S=5200, L=64, dtype=torch.bfloat16, seed=40 + r) for r in range(2)]
    pools = [pool_from_case(c)[0] for c in cases]
    group = LocalPeerGroup(pools, wait_polls=wait_polls)
    qs = [c.queries.cuda().reshape(c.num_streams, c.G, 128).contiguous() for c in cases]
    return cases, pools, group, qs


def _payload(recv, parity, j):
    """The rows rank j sent for `parity`, as they sit in a receive buffer: [R, 128] bf16 and the words' step counts."""
    words = recv[parity, j]  # [R, W, 2] int32
    data = words[..., 0].contiguous().view(torch.bfloat16).reshape(words.shape[0], 128)
    return data, words[..., 1]


def test_rows_land_in_every_ranks_buffer_with_parity_and_step_counts():
    cases, pools, group, qs = _two_ranks()
    R = pools[0].S * pools[0].G
    for step in range(1, 4):
        outs = []
        for r in range(2):
            q = (qs[r].float() * (1.0 + 0.05 * step)).to(torch.bfloat16)
            outs.append(pools[r].decode_step(q).clone())
        for r in range(2):
            group.wait(r)
        torch.cuda.synchronize()
        parity = (step - 1) & 1
        for r in range(2):
            assert not group.timed_out(r)
            assert int(group.seqs[r][0]) == step, "steps exchanged"
            buf = group.bufs[r]  # [2, world, R, 128]: row r' of rank j at ((parity * world + j) * R + r')
            for j in range(2):
                data, counts = _payload(group.recv[r], parity, j)
                assert bool((counts == step).all()), "every word of the step carries the step count"
                assert torch.equal(data, outs[j].reshape(R, 128)), f"step {step}: rank {j}'s words in rank {r}'s receive buffer"
                assert torch.equal(buf[parity, j], outs[j].reshape(R, 128)), f"step {step}: rank {j}'s rows gathered on rank {r}"
            assert torch.equal(group.result(r, step), buf[parity])
        if step >= 2:
            # the other parity still holds the previous step's rows: a rank one step ahead overwrites nothing a peer reads
            assert not torch.equal(group.bufs[0][parity], group.bufs[0][parity ^ 1])
            assert bool((group.recv[0][parity ^ 1, :, :, :, 1] == step - 1).all())


def test_the_wait_gives_up_and_the_context_stays_usable():
    """Rank 1 never steps: rank 0's receiving kernel runs out of polls for rank 1's words, reports it through the
    error flag and returns; the next step runs as usual.  Nothing hangs and nothing faults - the limit is a few
    thousand polls."""
    cases, pools, group, qs = _two_ranks(wait_polls=2000)
    R = pools[0].S * pools[0].G
    out0 = pools[0].decode_step(qs[0]).clone()
    group.wait(0)
    torch.cuda.synchronize()
    assert group.timed_out(0), "rank 1 sent nothing: the wait must report it"
    assert int(group.seqs[0][0]) == 1
    assert torch.equal(group.bufs[0][0, 0], out0.reshape(R, 128)), "rank 0's own rows were gathered"
    assert bool((group.bufs[0][0, 1] == 0).all()), "rank 1's rows were skipped"
    data, counts = _payload(group.recv[1], 0, 0)
    assert bool((counts == 1).all()) and torch.equal(data, out0.reshape(R, 128)), "rank 0's words still reached rank 1"
    # the stream and the context are intact: rank 1 steps, its wait succeeds
    group.seqs[0][1] = 0
    out1 = pools[1].decode_step(qs[1]).clone()
    group.wait(1)
    torch.cuda.synchronize()
    assert not group.timed_out(1)
    assert torch.equal(group.bufs[1][0, 1], out1.reshape(R, 128)) and torch.equal(group.bufs[1][0, 0], out0.reshape(R, 128))
    again = pools[0].decode_step(qs[0])
    torch.cuda.synchronize()
    assert float((again.float() - out0.float()).abs().max()) <= 1e-2 * float(out0.float().abs().max())


def test_wait_arguments_are_checked_on_the_host():
    import ctypes as C

    from pqhsa_release_b200 import _lib

    cases, pools, group, qs = _two_ranks()
    p = pools[0].p
    p.peer_wait_polls = -5
    with pytest.raises(_lib.PqhsaError):
        pools[0].decode_step(qs[0])
    p.peer_wait_polls = 0
    p.peer_rank = 7
    with pytest.raises(_lib.PqhsaError):
        _lib.call("pqhsa_wait_peers", C.byref(p), pools[0]._stream())
