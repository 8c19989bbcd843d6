"""The allocation-free classifier entry point (`sa_classify_mask_static`).

It exists for hosts that cannot allocate device memory at the point of the call - all memory
handed out at start-up, an allocator they are not allowed to touch, no latency budget for it - and
keeps its scratch in a fixed array inside the library.  Here it is called through the C ABI twice in
a row on different masks and must return exactly what the workspace-taking entry point returns
(integer lists: bit-exact).  The file is named so that it is collected last."""
import numpy as np
import pytest
import torch

import workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _outputs(nq, nk, S, fill):
    ids = lambda: torch.full((1, 1, nq, nk), fill, dtype=torch.int32, device=DEV)
    lens = lambda: torch.full((1, 1, nq), fill, dtype=torch.int32, device=DEV)
    bits = torch.full((1, 1, S // 32, S), fill, dtype=torch.int32, device=DEV)
    return ids(), lens(), ids(), lens(), bits


def test_static_scratch_entry_matches_workspace_entry(native_lib):
    S, bq, bk = 1024, 128, 32
    nq, nk = S // bq, S // bk
    stream = torch.cuda.current_stream().cuda_stream
    masks = [workloads.random_block_mask(1, S, 0.5, 0.2, seed=41).to(DEV).contiguous(),
             workloads.document_causal_mask(1, S, (100, 300), 0.1, seed=42).to(DEV).contiguous()]
    for call, m in enumerate(masks):                       # two calls in a row share the array
        want = _outputs(nq, nk, S, 7)
        ws_bytes = native_lib.sa_classify_workspace_bytes(1, 1, S, S)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
        rc = native_lib.sa_classify_mask(m.data_ptr(), 0, 0, S, 1, 1, 1, S, S, bq, bk,
                                         want[0].data_ptr(), want[1].data_ptr(), want[2].data_ptr(),
                                         want[3].data_ptr(), want[4].data_ptr(), ws.data_ptr(), ws_bytes,
                                         0, stream)          # 0: contents unknown, cleared by the call
        assert rc == 0
        got = _outputs(nq, nk, S, 9)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = native_lib.sa_classify_mask_static(m.data_ptr(), 0, 0, S, 1, 1, 1, S, S, bq, bk,
                                                got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(),
                                                got[3].data_ptr(), got[4].data_ptr(), stream)
        assert rc == 0, native_lib.sa_status_str(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        for name, a, b in zip(("full_ids", "full_lens", "part_ids", "part_lens", "bits"), got, want):
            assert np.array_equal(a.cpu().numpy(), b.cpu().numpy()), (call, name)
        assert int(got[1].sum()) + int(got[3].sum()) > 0


def test_static_scratch_entry_rejects_oversized_masks(native_lib):
    # one plane of 32768 x 32768 needs about half of the 1 MiB array; four planes do not fit
    S = 32768
    assert native_lib.sa_classify_workspace_bytes(1, 1, S, S) <= (1 << 20)
    need = native_lib.sa_classify_workspace_bytes(4, 1, S, S)
    assert need > (1 << 20)
    dummy = torch.zeros(64, dtype=torch.int32, device=DEV)
    p = dummy.data_ptr()
    rc = native_lib.sa_classify_mask_static(p, S * S, 0, S, 1, 4, 1, S, S, 128, 32, p, p, p, p, None,
                                            torch.cuda.current_stream().cuda_stream)
    assert rc == -3 and b"workspace" in native_lib.sa_status_str(rc)
