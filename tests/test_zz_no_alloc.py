"""The entry point for hosts that cannot allocate device memory (collected last on purpose).

``vtx_iir_fwd_noalloc`` keeps the carries between time segments in a scratch array that ships inside the
library instead of asking the caller for a buffer.  It must give exactly what ``vtx_iir_fwd`` gives with a
caller-provided buffer -- on the first call, and again on a second call that finds the first call's leftovers
in the shared array."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_noalloc_entry_point_matches_scratch_entry_point_twice():
    from vortex_b200 import _lib, ops

    B, L, D, G, S = 1, 6000, 32, 2, 16          # B*D is small, so the time axis is cut into segments (scratch in use)
    assert _lib.lib().vtx_iir_scratch_bytes(B, L, D, S, 0) > 0
    g = torch.Generator().manual_seed(123)
    log_poles = torch.log(0.9 + 0.099 * torch.rand(G, S, generator=g)).cuda()
    residues = torch.randn(G, S, generator=g).cuda()
    theta = (torch.pi * torch.rand(G, S, generator=g)).cuda()
    res_im = torch.randn(G, S, generator=g).cuda()
    for call, (dtype, cplx) in enumerate([(torch.float32, False), (torch.bfloat16, True)]):
        z = torch.randn(B, 3 * D, L, generator=g).to(dtype).cuda()
        bias = torch.randn(D, generator=g).to(dtype).cuda()
        kw = dict(theta=theta, res_im=res_im) if cplx else {}
        y_ref, st_ref = ops.iir_fwd(z, log_poles, residues, bias, D, **kw)
        y = torch.empty_like(y_ref)
        st = torch.empty_like(st_ref)
        ops.iir_fwd_noalloc(z, log_poles, residues, bias, D, y, st, **kw)
        torch.cuda.synchronize()
        assert torch.equal(y, y_ref), f"call {call}: outputs differ"
        assert torch.equal(st, st_ref), f"call {call}: states differ"


def test_noalloc_entry_point_refuses_sizes_beyond_its_scratch():
    from vortex_b200 import _lib, ops

    B, L, D, G, S = 1, 262144, 4096, 4096, 16     # complex poles: 4096 rows * 64 segments * 16 * 8 B = 32 MiB > 16 MiB built in
    assert _lib.lib().vtx_iir_scratch_bytes(B, L, D, S, 1) > 16 << 20
    # q / k / v / y stay NULL: the size check comes first, and should it ever regress the call still ends in the
    # null-pointer check instead of a launch that reads far outside a buffer
    p = _lib.IirParams(B=B, L=L, D=D, head_dim=D)
    p.modal.G, p.modal.S, p.modal.theta = G, S, 16      # theta is only compared with NULL (complex poles)
    import ctypes as C
    rc = _lib.lib().vtx_iir_fwd_noalloc(C.byref(p), None)
    assert rc == -2 and "built-in scratch" in _lib.last_error()
    with pytest.raises(NotImplementedError):
        _lib.check(rc)
