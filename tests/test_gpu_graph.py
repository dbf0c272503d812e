"""GPU: after one warm-up call has sized the per-stream scratch, sdq_qgemm makes no
allocation and no synchronisation, so a sequence of calls can be captured in a CUDA graph
(torch is used only to drive the capture) and replayed with identical results."""
import ctypes as C

import numpy as np
import pytest

from util import packed_weights

pytestmark = pytest.mark.gpu


def test_qgemm_calls_replay_from_a_cuda_graph(sdq, pkg, oracle):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(8)
    M, K, N = 192, 1024, 768
    A = rng.standard_normal((M, K)).astype(np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    want = oracle.qgemm(A, wq, ws)
    w = sdq.weight_upload(wq, ws)
    dA = torch.from_numpy(A).cuda()
    outs = [torch.zeros(M, N, device="cuda") for _ in range(6)]
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        sp = C.c_void_p(st.cuda_stream)
        sdq.qgemm(w, dA.data_ptr(), M, outs[0].data_ptr(), None, 0, sp)      # warm-up outside capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            for o in outs:
                sdq.qgemm(w, dA.data_ptr(), M, o.data_ptr(), None, 0, sp)
        for o in outs:
            o.zero_()
        graph.replay()
        torch.cuda.synchronize()
    for o in outs:
        assert o.cpu().numpy().tobytes() == want.tobytes()
    sdq.sync(None)
    sdq.weight_release(w)
