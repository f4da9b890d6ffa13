import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_ring_queue_serves_requests_in_order(runtime):
    """Ring_queue semantics (native/ocaml_metal_stubs.m:1465-1697): submit ->
    worker replays the plan -> completion {request_id, token, status}."""
    from llmopt_b200 import parameters
    from llmopt_b200.cuda_native import Buffer, DispatchItem, RingQueue

    token_buffer = Buffer.create(runtime, 8)
    output = Buffer.create(runtime, 8)
    ring = RingQueue()
    ring.start_worker(runtime, [DispatchItem("llmopt_chain_token_id", [token_buffer, output], b"", (32, 1, 1), (32, 1, 1))],
                      token_buffer, output)
    for request in range(5):
        assert ring.submit(request_id=request, token=100 + request, past_tokens=request)
    seen = [ring.wait_completion() for _ in range(5)]
    assert seen == [(request, 100 + request, 0) for request in range(5)]
    assert ring.poll_completion() is None
    ring.destroy()
