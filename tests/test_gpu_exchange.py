"""The peer-memory exchange + merge kernel (hira_exchange_merge) on one GPU: several emulated ranks
whose buffers all live on this device.  Their kernels must not wait on one another on one GPU, so
every rank first runs the push phase and then every rank runs the wait + merge phase; the fused
phase runs for a world of one, and on two GPUs in test_multi_gpu.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _partials(world, hq, v, seed):
    g = torch.Generator().manual_seed(seed)
    rows = torch.randn((world, hq, v + 2), generator=g)
    rows[:, :, 0] = rows[:, :, 0] * 5.0                      # running max m
    rows[:, :, 1] = rows[:, :, 1].abs() * 20.0 + 0.1         # denominator l
    rows[0, 0, 0] = float("-inf")                            # a shard that selected nothing for this head
    rows[0, 0, 1] = 0.0
    return rows.cuda()


@pytest.mark.parametrize("world,hq,v", [(4, 64, 128), (2, 8, 64), (8, 32, 128)])
def test_emulated_ranks_push_then_merge_equals_merge_partials(world, hq, v):
    from hira_b200 import _lib as L
    from hira_b200 import index_state as S
    from hira_b200.parallel import PeerPartialsExchange
    lib = L.load()
    nbytes = int(lib.hira_exchange_bytes(world, hq, v))
    assert nbytes == 2 * world * hq * ((v + 2) * 4 + 4)
    bufs = [torch.zeros((nbytes,), dtype=torch.uint8, device="cuda") for _ in range(world)]
    addrs = [b.data_ptr() for b in bufs]
    ranks = [PeerPartialsExchange(hq, v, "cuda", rank=r, world=world, peers=addrs) for r in range(world)]
    for step in range(1, 6):                                  # both parities, several times
        rows = _partials(world, hq, v, 100 + step)
        want = S.merge_partials(rows[:, :, 2:], rows[:, :, :2])
        want_ml = torch.empty((hq, 2), device="cuda")
        S.merge_partials(rows[:, :, 2:], rows[:, :, :2], out_ml=want_ml)
        for r, ex in enumerate(ranks):
            ex.local.copy_(rows[r])
            ex.merge(phases=1, seq=step, out=torch.empty((hq, v), device="cuda"))
        for r, ex in enumerate(ranks):
            got_ml = torch.empty((hq, 2), device="cuda")
            got = ex.merge(phases=2, seq=step, out_ml=got_ml)
            ex.check()
            assert torch.equal(got, want), (step, r)
            assert torch.equal(got_ml, want_ml), (step, r)


def test_world_of_one_fused_through_the_ipc_allocation():
    from hira_b200 import index_state as S
    from hira_b200.parallel import PeerPartialsExchange
    hq, v = 32, 128
    ex = PeerPartialsExchange(hq, v, "cuda")
    assert ex.world == 1 and ex.message_bytes == hq * (v + 2) * 4
    for step in range(3):
        rows = _partials(1, hq, v, 7 + step)
        ex.local.copy_(rows[0])
        got = ex.merge()
        ex.check()
        assert torch.equal(got, S.merge_partials(rows[:, :, 2:], rows[:, :, :2]))
    ex.close()
    ex.free()


def test_a_peer_that_never_pushes_ends_the_bounded_wait_with_a_status():
    """Rank 0 of an emulated world of two whose peer launches nothing: the wait (50 ms here) runs out,
    the status word is set, `out` keeps its content, and the context stays usable."""
    from hira_b200 import _lib as L
    from hira_b200.parallel import PeerPartialsExchange
    hq, v = 8, 64
    lib = L.load()
    nbytes = int(lib.hira_exchange_bytes(2, hq, v))
    bufs = [torch.zeros((nbytes,), dtype=torch.uint8, device="cuda") for _ in range(2)]
    ex = PeerPartialsExchange(hq, v, "cuda", rank=0, world=2, peers=[b.data_ptr() for b in bufs], wait_seconds=0.05)
    ex.local.copy_(_partials(1, hq, v, 3)[0])
    out = torch.full((hq, v), 7.0, device="cuda")
    ex.merge(out=out)
    with pytest.raises(RuntimeError, match="did not arrive"):
        ex.check()
    assert bool((out == 7.0).all())
    assert float(torch.ones(4, device="cuda").sum()) == 4.0   # the device still answers


def test_bad_arguments_are_refused_on_the_host():
    from hira_b200.parallel import PeerPartialsExchange
    with pytest.raises(ValueError):
        PeerPartialsExchange(8, 64, "cuda", rank=0, world=17, peers=[0] * 17)
    ex = PeerPartialsExchange(8, 64, "cuda")
    with pytest.raises(ValueError):
        ex.merge(seq=0)                                       # buffers start zeroed: step numbers start at 1
    ex.close()
    ex.free()
