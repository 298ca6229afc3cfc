"""GPU: the device status word on the operator path.  A kernel that gives up on a bounded wait sets
the word and every later CTA returns at once, so the operators poll it: the call after the failure
raises and clears it.  The failure is made without any fault or hang: the word is set from the host,
or by the library's self-test kernel, whose wait (50 microseconds) on a barrier that nothing
completes runs out and leaves through the attention kernel's tear-down."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from dfsattn_b200 import ops
    torch.cuda.synchronize()
    ops.status_tensor("cuda").zero_()
    yield
    torch.cuda.synchronize()
    ops.status_tensor("cuda").zero_()
    try:
        ops.check_status("cuda")
    except RuntimeError:
        pass


def _small_call():
    from dfsattn_b200.attention_hyvideo import dfs_attention
    from dfsattn_b200.synthetic import structured_qkv
    q, k, v = structured_qkv((2, 8, 16), 2, 128, dtype=torch.bfloat16, device="cuda", seed=5)
    kw = dict(step_idx=12, skip_steps=12, cache_interval=12, layer_idx=77, sparsity=0.5, sparsity_dcrt=0.1,
              tile_size=16, block_size=128, video_len=256, video_perm=None)
    return lambda: dfs_attention(q, k, v, **kw)


def test_bounded_wait_runs_out_and_reports():
    from dfsattn_b200 import ops
    from dfsattn_b200._lib import check, lib
    word = ops.status_tensor("cuda")
    check(lib.dfs_selftest_wait_timeout(100_000, word.data_ptr(), torch.cuda.current_stream().cuda_stream),
          "dfs_selftest_wait_timeout")
    torch.cuda.synchronize()
    assert int(word.item()) == 1                      # DFS_STATUS_WAIT_TIMEOUT
    with pytest.raises(RuntimeError, match="bounded wait"):
        ops.check_status("cuda")
    ops.check_status("cuda")                          # cleared by the raise
    with pytest.raises(ValueError):
        check(lib.dfs_selftest_wait_timeout(0, word.data_ptr(), None), "dfs_selftest_wait_timeout")
    with pytest.raises(ValueError):
        check(lib.dfs_selftest_wait_timeout(1000, None, None), "dfs_selftest_wait_timeout")


@pytest.mark.parametrize("how", ["host", "kernel"])
def test_operator_raises_one_call_after_a_give_up(how):
    from dfsattn_b200 import ops
    from dfsattn_b200._lib import check, lib
    from dfsattn_b200.attention_hyvideo import DFS_Attention
    call = _small_call()
    good = call().clone()
    torch.cuda.synchronize()
    word = ops.status_tensor("cuda")
    if how == "host":
        word.fill_(1)
    else:
        check(lib.dfs_selftest_wait_timeout(100_000, word.data_ptr(), torch.cuda.current_stream().cuda_stream),
              "dfs_selftest_wait_timeout")
    call()                                            # its kernels see the word and do nothing; no error yet
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="device status 1"):
        call()                                        # the poll of this call reads what the last one copied
    torch.cuda.synchronize()
    assert int(word.item()) == 0                      # cleared
    again = call()
    torch.cuda.synchronize()
    assert torch.equal(again, good)                   # and the operator works again
    ops.check_status("cuda")
    DFS_Attention.clear_cache()


def test_dense_call_polls_too():
    from dfsattn_b200 import ops
    from dfsattn_b200.fullattention import full_attention
    q = torch.randn(1, 2, 256, 128, device="cuda", dtype=torch.bfloat16)
    full_attention(q, q, q, mode="flash")
    torch.cuda.synchronize()
    ops.status_tensor("cuda").fill_(2)
    full_attention(q, q, q, mode="flash")
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="device status 2"):
        full_attention(q, q, q, mode="flash")
