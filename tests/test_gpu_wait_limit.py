"""A bounded device-side wait that runs out is counted, leaves the context usable and is reported by
the host.  Runs in a child process so that the library's counter never leaks into other tests."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import math, sys, torch
    sys.path.insert(0, %r)
    from shareprefill_b200 import native
    lib = native.load()
    assert native.device_timeouts() == 0
    # a 2 ms limit, then a kernel whose only wait is on a barrier nothing ever arrives on
    assert lib.spf_set_device_wait_limit_ns(2_000_000) == 0
    assert lib.spf_wait_limit_selftest(torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()                      # the kernel returned by itself
    assert native.device_timeouts() == 1, native.device_timeouts()
    try:
        native.raise_on_device_timeouts()
    except native.SpfError as e:
        assert "gave up" in str(e)
    else:
        raise AssertionError("the host did not report the timeout")
    assert native.device_timeouts() == 0          # reporting clears the counter
    # the context is intact: a real kernel runs and waits normally with the default limit restored
    assert lib.spf_set_device_wait_limit_ns(1_000_000_000) == 0
    g = torch.Generator().manual_seed(0)
    q = torch.randn(512, 2, 128, generator=g).bfloat16().cuda()
    k = torch.randn(512, 1, 128, generator=g).bfloat16().cuda()
    v = torch.randn(512, 1, 128, generator=g).bfloat16().cuda()
    full = native.sets_to_bitmap([torch.tensor([r * 4 + c for r in range(4) for c in range(r + 1)])] * 2, 4, "cuda")
    out = native.sparse_attention(q, k, v, full, 128, 1 / math.sqrt(128))
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], is_causal=True,
        enable_gqa=True)[0].transpose(0, 1)
    err = (out.float() - ref.float()).abs()
    assert bool((err <= torch.maximum(torch.full_like(err, 2e-2), ref.float().abs() * 2.0 ** -7)).all())
    assert native.device_timeouts() == 0
    # more than 16 recorded timeouts: the tcgen05 entry points refuse to launch until the counter is reset
    assert lib.spf_set_device_wait_limit_ns(200_000) == 0
    for _ in range(17):
        lib.spf_wait_limit_selftest(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert native.device_timeouts() == 17
    try:
        native.sparse_attention(q, k, v, full, 128, 1 / math.sqrt(128))
    except native.SpfError as e:
        assert "(-7)" in str(e)
    else:
        raise AssertionError("launch was not refused")
    assert lib.spf_reset_device_timeouts() == 0 and native.device_timeouts() == 0
    native.sparse_attention(q, k, v, full, 128, 1 / math.sqrt(128))
    torch.cuda.synchronize()
    print("wait-limit ok")
""") % ROOT


def test_wait_that_runs_out_is_counted_and_reported():
    res = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "wait-limit ok" in res.stdout
