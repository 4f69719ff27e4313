"""fdma_fwd_static_scratch -- the forward entry point for hosts that cannot provide scratch memory (engines with
device memory carved up at start-up and no allocator for operators, loops where an allocation is unacceptable).
The built-in array serves whatever fdma_fwd_workspace_bytes asks for: the tile-activity bytes of a per-query mask, or
the split partials of a single-query (decode) call.

Called through the C ABI, twice in a row with different per-query masks (so the second call runs on top of the
first call's left-over scratch contents), and compared with fdma_fwd given caller-allocated scratch. Same kernels,
same inputs, deterministic forward: the outputs must be identical. The file name keeps this test last in
collection order."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _params(lib_mod, iface, q, k, v, mask, bias, out, lse, causal):
    p = lib_mod.FwdParams()
    iface._fill_fwd(p, q, k, v, mask, bias, out, lse, q.shape[-1] ** -0.5, causal)
    return p


def test_static_scratch_matches_caller_scratch_on_two_consecutive_calls():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from flash_sparse_attn import _lib
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    lib = _lib.load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    B, Sq, Sk, H, Hk, d = 2, 384, 512, 4, 2, 128
    g = torch.Generator().manual_seed(11)
    q = torch.randn((B, Sq, H, d), generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn((B, Sk, Hk, d), generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn((B, Sk, Hk, d), generator=g).to(torch.bfloat16).to(dev)
    bias = torch.randn((B, Hk, Sq, Sk), generator=g).to(torch.bfloat16).to(dev)
    masks = []
    for density in (0.3, 0.02):  # the second mask empties many 128x128 tiles that the first one kept
        m = torch.rand((B, Hk, Sq, Sk), generator=g) < density
        m[:, :, :128, 256:] = density > 0.1  # whole tiles that flip between the two calls
        masks.append(m.to(dev))

    assert lib.fdma_static_scratch_limit() == 1 << 20
    for mask in masks:
        out_ref = torch.full_like(q, float("nan"))
        lse_ref = torch.empty((B, H, Sq), dtype=torch.float32, device=dev)
        p = _params(_lib, iface, q, k, v, mask, bias, out_ref, lse_ref, True)
        need = lib.fdma_fwd_workspace_bytes(ctypes.byref(p))
        assert need > 0, "this case must be one that uses scratch"
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        p.workspace, p.workspace_bytes = ws.data_ptr(), need
        assert lib.fdma_fwd(ctypes.byref(p), stream) == 0

        out_new = torch.full_like(q, float("nan"))
        lse_new = torch.empty_like(lse_ref)
        p2 = _params(_lib, iface, q, k, v, mask, bias, out_new, lse_new, True)  # no workspace given
        assert lib.fdma_fwd_static_scratch(ctypes.byref(p2), stream) == 0
        torch.cuda.synchronize()
        assert torch.isfinite(out_new.float()).all()
        assert torch.equal(out_new, out_ref)
        assert torch.equal(lse_new, lse_ref)

    # a problem whose scratch exceeds the built-in array is refused before anything is launched
    big = _params(_lib, iface, q, k, v, masks[0], bias, out_new, lse_new, True)
    big.b, big.h, big.h_k, big.h_mask, big.h_bias = 64, 32, 32, 32, 32
    big.seqlen_q = big.seqlen_k = 8192
    assert lib.fdma_fwd_workspace_bytes(ctypes.byref(big)) > lib.fdma_static_scratch_limit()
    assert lib.fdma_fwd_static_scratch(ctypes.byref(big), stream) == -7
    assert b"static scratch" in lib.fdma_strerror(-7)
    torch.cuda.synchronize()


def test_static_scratch_serves_single_query_calls_up_to_its_limit():
    """A single-query forward keeps its per-split partials (B, H, splits x 8 warps, d + 2) fp32 in scratch, whether or
    not there is a mask: a call whose partials fit the 1 MiB array equals fdma_fwd bit for bit (twice in a row), one
    whose partials do not fit is refused with FDMA_ERR_TOO_LARGE before anything is launched."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from flash_sparse_attn import _lib
    from flash_sparse_attn import flash_sparse_attn_interface as iface

    lib = _lib.load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    g = torch.Generator().manual_seed(23)
    Sk, H, Hk, d = 3000, 8, 2, 128
    for B, fits in ((4, True), (4, True), (64, False)):
        q = torch.randn((B, 1, H, d), generator=g).to(torch.bfloat16).to(dev)
        k = torch.randn((B, Sk, Hk, d), generator=g).to(torch.bfloat16).to(dev)
        v = torch.randn((B, Sk, Hk, d), generator=g).to(torch.bfloat16).to(dev)
        bias = torch.randn((B, Hk, 1, 3072), generator=g).to(torch.bfloat16).to(dev)
        mask = (torch.rand((B, Hk, 1, 3072), generator=g) < 0.25).to(dev)
        out_ref = torch.full_like(q, float("nan"))
        lse_ref = torch.empty((B, H, 1), dtype=torch.float32, device=dev)
        p = _params(_lib, iface, q, k, v, mask, bias, out_ref, lse_ref, False)
        need = lib.fdma_fwd_workspace_bytes(ctypes.byref(p))
        assert need > 0
        assert (need <= lib.fdma_static_scratch_limit()) == fits, need
        out_new = torch.full_like(q, float("nan"))
        lse_new = torch.empty_like(lse_ref)
        p2 = _params(_lib, iface, q, k, v, mask, bias, out_new, lse_new, False)
        if not fits:
            assert lib.fdma_fwd_static_scratch(ctypes.byref(p2), stream) == -7
            continue
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        p.workspace, p.workspace_bytes = ws.data_ptr(), need
        assert lib.fdma_fwd(ctypes.byref(p), stream) == 0
        assert lib.fdma_fwd_static_scratch(ctypes.byref(p2), stream) == 0
        torch.cuda.synchronize()
        assert torch.isfinite(out_new.float()).all()
        assert torch.equal(out_new, out_ref) and torch.equal(lse_new, lse_ref)
