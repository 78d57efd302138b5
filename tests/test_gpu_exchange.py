"""Expert-parallel exchange over peer memory, on one GPU.

The kernels that move the kept lists and the partial output rows between ranks
(`cfm_select`, `cfm_adopt` and `cfm_partial_output` with an exchange,
`cfm_finish_rows`) run here with a group of one rank: the rank stores into its own
block, so every flag a kernel waits for has been set by an earlier kernel of the
same stream and no launch ever waits on another.  Two ranks over NVLink are
covered by tests/test_gpu_expert_parallel.py.

The bounded wait is tested the way a lost rank would look from the device: a
finish on a fresh block, whose flags nothing sets, gives up after about a second
and reports it in the status word; the context stays usable.
"""

import ctypes
import socket

import pytest
import torch
import torch.distributed as dist

from cfm_b200 import _native
from helpers import prepared
from test_gpu_parity import _channel_major, _move_statistics, make_reader, run_reader

pytestmark = pytest.mark.gpu


@pytest.fixture()
def one_rank_group():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                            device_id=device)
    try:
        yield device
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name", ["qwen35-e16-t4", "qwen3-e16-t8", "graph-routes"])
def test_one_rank_exchange_matches_the_single_gpu_reader(one_rank_group, name):
    from cfm_b200.reader.expert_parallel import ExpertParallelReader

    device = one_rank_group
    item = prepared(name)
    case = item["case"]
    whole = make_reader(item)
    expected = run_reader(whole, case).clone()
    tokens = case.hidden.shape[0]
    sharded = ExpertParallelReader(
        case.gate_up.to(device), _channel_major(item["down"], device),
        case.encoder.to(device) if case.encoder is not None else None,
        case.decoder.to(device) if case.decoder is not None else None,
        case.plan, tokens, global_experts=case.gate_up.shape[0], exchange="peer",
        sketch=(item["codes"].to(device), _move_statistics(item["statistics"], device)),
        activation=case.activation, selection_score=case.score,
    )
    assert sharded.exchange is not None and sharded.exchange.available
    padding = case.padding.to(device) if case.padding is not None else None
    inputs = (case.hidden.to(device), case.ids.to(device), case.weights.to(device), padding)
    active = ~case.padding if case.padding is not None else torch.ones(tokens, dtype=torch.bool)
    for _ in range(3):  # three epochs of the exchange
        out = sharded(*inputs)
        torch.cuda.synchronize()
        assert torch.equal(sharded.home.workspace.candidate_ids[:tokens][active],
                           whole.candidate_ids[-1][:tokens][active])
        assert torch.equal(out[active], expected[active])
        assert not out[~active].any()
    # The same through a captured graph, replayed twice.
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            captured = sharded(*inputs)
        for _ in range(2):
            graph.replay()
        stream.synchronize()
    assert torch.equal(captured[active], expected[active])
    assert sharded.exchange.status() == 0


def test_a_wait_that_nothing_ends_gives_up_and_reports(one_rank_group):
    from cfm_b200.reader.expert_parallel import PeerExchange

    device = one_rank_group
    item = prepared("graph-routes")
    reader = make_reader(item)
    tokens = 2
    exchange = PeerExchange(reader._layer, tokens, dist.group.WORLD)
    assert exchange.available and exchange.status() == 0
    out = torch.zeros(tokens, item["case"].plan.hidden_size, device=device, dtype=torch.bfloat16)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    code = _native.load().cfm_finish_rows(
        ctypes.byref(reader._layer), ctypes.byref(exchange.struct), None, out.data_ptr(),
        ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream))
    end.record()
    assert code == 0
    torch.cuda.synchronize()
    assert exchange.status() & 2  # the rows of the only rank never arrived
    assert 100 < start.elapsed_time(end) < 10_000  # about a second, not forever
    # The context is still usable and the reader still works.
    again = run_reader(reader, item["case"])
    assert torch.isfinite(again.float()).all()
