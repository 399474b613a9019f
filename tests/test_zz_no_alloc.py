"""The allocation-free decode entry point against the regular one.

Some hosts of this library cannot allocate device memory at the moment they call it: a server
that reserved all memory at start-up and treats a later cudaMalloc as a bug, a latency-critical loop
that cannot take an allocation's implicit synchronisation, or a plugin interface that only passes
input and output buffers.  For them
`kvskip_launch_decode_noalloc` keeps the split-K partials in an array built into the library.
This test drives it through the C ABI (ctypes), twice in a row on the same buffers, and expects
the same bits as `kvskip_launch_decode` with caller-provided scratch -- it is the same kernel, only
the scratch differs.  The file sorts last so a run that stops at the first failure has already run
everything else.
"""
import pytest
import torch

from kvskip_b200 import synth
from kvskip_b200.cabi import CAbi

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_noalloc_matches_regular_entry_point_twice():
    abi = CAbi()
    q, k, v, scale, keep = synth.sink_body_case(5, T=4096 + 40, B=2)
    qc, kc, vc = q.to(DEV), k.to(DEV), v.to(DEV)
    bi, bc = synth.keep_to_plan(keep)
    bi, bc = bi.to(DEV), bc.to(DEV)
    out = torch.empty(2, 32, 128, dtype=torch.bfloat16, device=DEV)
    o32 = torch.empty(2, 32, 128, dtype=torch.float32, device=DEV)
    lse = torch.empty(2, 32, dtype=torch.float32, device=DEV)
    for kw in (dict(), dict(block_idx=bi, block_cnt=bc)):
        for splits in (6, 1):
            ref = abi.decode(qc, kc, vc, scale, num_splits=splits, want_f32=True, **kw)
            # first call of a configuration: kernel attributes, the scratch address (set-up, may touch memory)
            abi.decode_noalloc(qc, kc, vc, scale, out, lse, num_splits=splits, out_f32=o32, **kw)
            torch.cuda.synchronize()
            for call in range(2):
                out.fill_(0), o32.fill_(0), lse.fill_(0)
                torch.cuda.synchronize()
                # free device memory as the driver reports it: sees a cudaMalloc inside the library,
                # which the framework's own allocator statistics would not
                free_before = torch.cuda.mem_get_info()[0]
                before = torch.cuda.memory_allocated()
                abi.decode_noalloc(qc, kc, vc, scale, out, lse, num_splits=splits, out_f32=o32, **kw)
                torch.cuda.synchronize()
                assert torch.cuda.mem_get_info()[0] == free_before
                assert torch.cuda.memory_allocated() == before
                assert torch.equal(out, ref[0]), (kw.keys(), splits, call)
                assert torch.equal(lse, ref[1]) and torch.equal(o32, ref[4])


def test_noalloc_rejects_oversized_scratch():
    abi = CAbi()
    q, k, v, scale = synth.dense_case(6, 4, 1024)
    qc, kc, vc = q.to(DEV), k.to(DEV), v.to(DEV)
    out = torch.empty(4, 32, 128, dtype=torch.bfloat16, device=DEV)
    lse = torch.empty(4, 32, dtype=torch.float32, device=DEV)
    with pytest.raises(RuntimeError, match="exceed"):
        abi.decode_noalloc(qc, kc, vc, scale, out, lse, num_splits=64)      # 4*32*64*130 floats > 1 Mi
