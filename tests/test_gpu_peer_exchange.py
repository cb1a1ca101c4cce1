"""The in-kernel head-output exchange, exercised on one GPU.

The peers' buffers and arrival counters are ordinary device memory here: the
stores, the unit counting, the once-per-call signal and the bounded wait are the
same code that runs across GPUs (where the buffers are peer mappings).
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from community_kv_b200 import native, ops
from community_kv_b200.config import CommunityKVConfig
from community_kv_b200.runtime import convert_prefill_tensors
from community_kv_b200.state import DecodeLayerWorkspace
from community_kv_b200.synthetic import make_layer, make_query

pytestmark = pytest.mark.gpu
SCALE = 128 ** -0.5


def _layer_args(device, *, splits, aggregation="query_group"):
    layer = make_layer(seed=70, kv_heads=4, seq_len=4096, communities=64, max_decode_tokens=4,
                       aggregation=aggregation)
    converted = convert_prefill_tensors(**layer.to(device).prepare_kwargs())
    heads = converted.mutable.retrieval_head_count
    workspace = DecodeLayerWorkspace.allocate(
        retrieval_head_count=heads, graph_count=converted.mutable.graph_count, group_size=converted.group_size,
        community_capacity=converted.mutable.community_capacity, token_budget=512, num_sink=6,
        dtype=torch.bfloat16, device=device, splits=splits,
    )
    query = make_query(seed=71, query_heads=layer.query_heads).to(device)
    args = ops.build_layer_args(
        query=query, key=layer.key.to(device), value=layer.value.to(device), csr=converted.csr,
        state=converted.mutable, sink_positions=torch.arange(6, dtype=torch.int32, device=device),
        current_position=converted.current_position, softmax_scale=SCALE, lam=0.5, workspace=workspace,
    )
    return args, workspace, (layer, converted, query)


@pytest.mark.parametrize("unfused", [False, True])
def test_merge_phase_stores_rows_to_peers_and_signals_once(unfused):
    device = torch.device("cuda", 0)
    args, workspace, keep = _layer_args(device, splits=4)
    if unfused:
        args.flags |= native.FLAG_UNFUSED
    assert native.library().ckv_decode_layer_kernels(ctypes.byref(args)) == (4 if unfused else 1)
    output = workspace.attention.output
    peers = [torch.zeros_like(output) for _ in range(3)]
    flags = torch.zeros((3,), dtype=torch.int32, device=device)
    done = torch.zeros((1,), dtype=torch.int32, device=device)
    status = torch.zeros((1,), dtype=torch.int32, device=device)
    args.peer_count = 3
    for index, peer in enumerate(peers):
        args.peer_output[index] = peer.data_ptr()
        args.peer_flag[index] = flags.data_ptr() + 4 * index
    args.peer_done = done.data_ptr()
    stream = native.current_stream(device)
    native.call("ckv_decode_layer", args, stream)
    lib = native.library()
    for index in range(3):  # one arrival per peer and call, however many units there are
        assert lib.ckv_wait_peers(ctypes.c_void_p(flags.data_ptr() + 4 * index), ctypes.c_uint32(1),
                                  ctypes.c_void_p(status.data_ptr()), ctypes.c_void_p(stream)) == 0
    torch.cuda.synchronize(device)
    assert int(status.item()) == 0
    assert flags.tolist() == [0, 0, 0] and int(done.item()) == 0  # counts taken back off
    for peer in peers:
        assert torch.equal(peer, output)
    del keep


def test_wait_for_peers_gives_up_and_reports():
    """A counter nobody increments: the bounded wait returns, sets the status word, and the
    context stays usable."""

    device = torch.device("cuda", 0)
    flag = torch.zeros((1,), dtype=torch.int32, device=device)
    status = torch.zeros((1,), dtype=torch.int32, device=device)
    stream = native.current_stream(device)
    lib = native.library()
    assert lib.ckv_wait_peers(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint32(1),
                              ctypes.c_void_p(status.data_ptr()), ctypes.c_void_p(stream)) == 0
    torch.cuda.synchronize(device)
    assert int(status.item()) & 1 == 1  # CKV_DEV_WAIT_TIMEOUT
    assert int(flag.item()) == 0
    assert float((torch.ones(4, device=device) * 2).sum()) == 8.0
    assert lib.ckv_wait_peers(None, ctypes.c_uint32(1), None, ctypes.c_void_p(stream)) < 0
