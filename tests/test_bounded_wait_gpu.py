"""The error path of the bounded waits, on one GPU and without any fault: the wait budget is shortened to about a
millisecond, a kernel is made to wait on a flag that nothing sets, and the host reads the status word.  The context
stays usable: the same kernels give correct results afterwards."""
import pytest
import torch

pytestmark = pytest.mark.gpu

STATUS_TIMEOUT_PEER_FLAG = 5
STATUS_TIMEOUT_LOCAL_FLAG = 7


@pytest.fixture
def short_waits():
    from litetorch_b200.ops import kernels as K
    K.status_fetch()
    K.set_wait_budget(2_000_000, 2_000_000)          # ~1 ms at 1.9 GHz
    yield K
    torch.cuda.synchronize()
    K.set_wait_budget(0, 0)                           # defaults
    K.status_fetch()


def test_barrier_whose_peer_never_arrives_reports_and_returns(short_waits):
    K = short_waits
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")
    other = torch.zeros(64, dtype=torch.int32, device="cuda")      # stands in for rank 1's flag words; rank 1 does not exist
    K.signal_barrier(mine, [mine.data_ptr(), other.data_ptr()], 0, 1, 2, 0)
    assert K.status_fetch() == STATUS_TIMEOUT_PEER_FLAG
    assert int(mine[0]) == 1 and int(other[0]) == 1                # this rank's own signals were delivered
    assert int(mine[1]) == 0                                       # the word the absent rank would have written
    # the context is intact: a GEMM right after gives the right answer, and the status word is clean again
    a = torch.randn(256, 128, device="cuda").bfloat16()
    b = torch.randn(192, 128, device="cuda").bfloat16()
    c = K.gemm(a, b)
    ref = a.float() @ b.float().t()
    assert float((c.float() - ref).abs().max() / ref.abs().max()) < 2e-2
    assert K.status_fetch() == 0


def test_gemm_reduce_scatter_with_a_silent_peer_times_out_cleanly(short_waits):
    """GEMM -> reduce-scatter for a world of two in which only rank 0 runs: its tiles are computed and sent, the
    reduce phase waits for the second contribution to its own rows, gives up, frees tensor memory and returns."""
    K = short_waits
    M, N, Kd = 256, 256, 128
    a = torch.randn(M, Kd, device="cuda").bfloat16()
    b = torch.randn(N, Kd, device="cuda").bfloat16()
    stage = [torch.zeros(M * N, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    counters = [torch.zeros(4096, dtype=torch.int32, device="cuda") for _ in range(2)]
    K.gemm_rs(a, b, b_major=0, stage_ptrs=[s.data_ptr() for s in stage], counter_ptrs=[c.data_ptr() for c in counters],
              epoch=1, world=2, rank=0)
    st = K.status_fetch()
    assert st in (STATUS_TIMEOUT_PEER_FLAG, STATUS_TIMEOUT_LOCAL_FLAG), st
    # afterwards the same kernel in a world of one (nobody to wait for) is correct: tensor memory was released
    stage1 = torch.zeros(M * N, dtype=torch.bfloat16, device="cuda")
    counters1 = torch.zeros(4096, dtype=torch.int32, device="cuda")
    out = K.gemm_rs(a, b, b_major=0, stage_ptrs=[stage1.data_ptr()], counter_ptrs=[counters1.data_ptr()], epoch=1, world=1, rank=0)
    ref = a.float() @ b.float().t()
    assert float((out.float() - ref).abs().max() / ref.abs().max()) < 2e-2
    assert K.status_fetch() == 0
