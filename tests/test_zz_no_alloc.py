"""bpsn_gae_static -- the GAE entry point for callers that cannot allocate.

A trainer that fixed its GPU memory budget at start-up (or any host whose allocator belongs to
another runtime) cannot hand `bpsn_gae` the device workspace it asks for.  `bpsn_gae_static`
keeps that scratch in a fixed array inside the library, so the call allocates nothing.  This test
goes through the C ABI directly (ctypes, raw device pointers), runs the static variant twice in a
row on different inputs, and requires each result to equal what `bpsn_gae` (caller workspace)
produces for the same inputs -- within the tolerances the other GAE tests use; in practice the two
run the same kernels and agree bit for bit.  It also checks that a batch beyond the built-in limit
is refused with an error rather than overrunning the array.

The file name sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _inputs(T, N, seed, pdone):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rewards = torch.randn(T + 1, N, 1, device="cuda", generator=g)
    values = torch.randn(T + 1, N, 1, device="cuda", generator=g)
    masks = (torch.rand(T + 1, N, 1, device="cuda", generator=g) >= pdone)
    next_value = torch.randn(N, 1, device="cuda", generator=g)
    return rewards, values, masks, next_value


def _run(lib, static, rewards, values, masks, next_value, T, N, normalize):
    from bps_nav_b200 import _lib as L
    values = values.clone()
    returns = torch.zeros_like(rewards)
    adv = torch.empty(T, N, 1, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    common = [rewards.data_ptr(), values.data_ptr(), masks.data_ptr(), next_value.data_ptr(),
              returns.data_ptr(), adv.data_ptr(), T, N, 0.99, 0.95, 1 if normalize else 0, 1e-5]
    if static:
        L.check(lib.bpsn_gae_static(*common, stream))
    else:
        ws = torch.empty(lib.bpsn_gae_workspace_bytes(N), dtype=torch.uint8, device="cuda")
        L.check(lib.bpsn_gae(*common, ws.data_ptr(), stream))
    torch.cuda.synchronize()
    return returns.cpu().numpy(), adv.cpu().numpy(), values.cpu().numpy()


def test_static_gae_matches_workspace_gae_twice():
    from bps_nav_b200 import _lib as L
    lib = L.load()
    # two calls in a row, different shapes and contents: the second must not see the first's scratch
    for call, (T, N, seed, pdone) in enumerate([(32, 16384, 11, 0.002), (16, 1000, 12, 0.05)]):
        rewards, values, masks, nv = _inputs(T, N, seed, pdone)
        for normalize in (True, False):
            ref = _run(lib, False, rewards, values, masks, nv, T, N, normalize)
            got = _run(lib, True, rewards, values, masks, nv, T, N, normalize)
            for name, a, b in zip(("returns", "advantages", "values"), got, ref):
                assert np.allclose(a[:T], b[:T], rtol=1e-5, atol=2e-6), \
                    f"call {call}, normalize={normalize}: {name} differ"
            assert np.array_equal(got[0][:T], ref[0][:T])
            if call == 0:
                # and against the CPU oracle, not only against the sibling entry point
                from oracle import pyoracle
                o_ret, o_adv, _ = pyoracle.gae_reference(
                    rewards[..., 0].cpu().numpy(), values[..., 0].cpu().numpy(),
                    masks[..., 0].cpu().numpy(), nv[:, 0].cpu().numpy(), 0.99, 0.95,
                    normalize=normalize)
                assert np.allclose(got[0][:T, :, 0], o_ret[:T], rtol=1e-5, atol=1e-6)
                assert np.allclose(got[1][..., 0], o_adv, rtol=1e-5, atol=2e-6)


def test_static_gae_leaves_device_memory_alone():
    """The point of the entry point: the call itself must not take or return device memory.
    Free memory as the driver reports it is the same before and after."""
    from bps_nav_b200 import _lib as L
    lib = L.load()
    T, N = 32, 16384
    rewards, values, masks, nv = _inputs(T, N, 21, 0.002)
    returns = torch.zeros_like(rewards)
    adv = torch.empty(T, N, 1, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call():
        L.check(lib.bpsn_gae_static(rewards.data_ptr(), values.data_ptr(), masks.data_ptr(),
                                    nv.data_ptr(), returns.data_ptr(), adv.data_ptr(), T, N,
                                    0.99, 0.95, 1, 1e-5, stream))

    # The set-up call comes first (documented: the first call on a device resolves the array's
    # address; the CUDA runtime also loads the two kernels' code at their first launch, which
    # is the runtime's memory, not this library's).
    call()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0


def test_static_gae_rejects_oversize_batch():
    from bps_nav_b200 import _lib as L
    lib = L.load()
    T, N = 1, 262144 + 1
    # sizes are validated before anything is launched, so tiny dummy buffers are enough
    dummy = torch.zeros(16, device="cuda")
    rc = lib.bpsn_gae_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None,
                             dummy.data_ptr(), dummy.data_ptr(), T, N, 0.99, 0.95, 0, 1e-5, None)
    assert rc == L.ERR_INVALID_ARG
    assert b"exceeds" in lib.bpsn_last_error(None)
