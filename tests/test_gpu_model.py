"""A whole Hugging Face decoder through the plug-in: prefill kernel -> partitioner -> decode kernels.

A small random-init Qwen3-shaped model (two layers, 8 query / 2 KV heads, head_dim 128) runs
``CommunityKVRuntime.generate`` with ``CommunityKVAttention`` registered as its attention
function, as the reference is used (community_kv/runtime.py:510-608, attention/adapter.py:33-81):
the prompt goes through the fused prefill kernel, its neighbour edges are handed to a (synthetic)
host partitioner, the static cache is switched to device-side cursors, and every further token
runs one decode-layer call per layer.  The same weights with dense attention are the reference:
with a prompt of 255 tokens the effective budget is 256, so the first decode step retrieves
every cached token and must reproduce the dense logits; later steps are sparse and are checked
for finiteness, cursor and label bookkeeping.
"""

from __future__ import annotations

import pytest
import torch

from community_kv_b200 import CommunityKVAttention, CommunityKVConfig, CommunityKVRuntime, PartitionConfig
from community_kv_b200.synthetic import SyntheticPartitioner

pytestmark = pytest.mark.gpu


def _tiny_model(device):
    from transformers import Qwen3Config, Qwen3ForCausalLM

    torch.manual_seed(0)
    config = Qwen3Config(
        hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=8,
        num_key_value_heads=2, head_dim=128, vocab_size=512, max_position_embeddings=4096,
        tie_word_embeddings=False,
    )
    model = Qwen3ForCausalLM(config).to(device=device, dtype=torch.bfloat16).eval()
    return model


@pytest.mark.parametrize("aggregation", ["query_group", "per_query_head"])
def test_generate_through_the_plugin_matches_dense_attention(aggregation):
    device = torch.device("cuda", 0)
    model = _tiny_model(device)
    prompt_length, new_tokens = 255, 6
    generator = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 512, (1, prompt_length), generator=generator).to(device)

    model.config._attn_implementation = "sdpa"
    with torch.no_grad():
        dense = model.generate(prompt, max_new_tokens=new_tokens, do_sample=False, output_scores=True,
                               return_dict_in_generate=True)

    config = CommunityKVConfig(token_budget=1024, num_sink=4, lam=0.5, aggregation=aggregation)
    partitioner = SyntheticPartitioner(communities=24, zipf_exponent=1.1, seed=3)
    with CommunityKVRuntime(config=config, partition=PartitionConfig(), num_layers=2,
                            max_decode_tokens=new_tokens, partitioner=partitioner) as runtime:
        name = CommunityKVAttention(runtime).register()
        model.config._attn_implementation = name
        with torch.no_grad():
            sparse = runtime.generate(model, prompt, max_new_tokens=new_tokens, output_scores=True,
                                      return_dict_in_generate=True)
        runtime.assert_no_overflow()
        # both layers went through the prefill kernel and handed their edges to the partitioner
        assert set(partitioner.edges_seen) == {0, 1}
        assert partitioner.edges_seen[0] == (8, prompt_length - (4 + 7), 8)
        # ... which coalesced them into a graph (direct and co-attention edges of 244 rows per head)
        assert all(edges > 244 * 8 for edges in partitioner.adjacency_edges.values())
        for layer in runtime.decode_runtime.layers.values():
            assert layer.workspace.selection.token_budget == 256
            steps = new_tokens - 1  # the first new token comes out of the prefill
            assert int(layer.converted.current_position.min()) == prompt_length + steps
            labels = layer.converted.mutable.token_communities[:, prompt_length : prompt_length + steps]
            assert int(labels.min()) >= 0

    # token 0: prefill logits (dense causal attention in the prefill kernel);
    # token 1: first decode step, every cached token retrieved
    for step in (0, 1):
        got, want = sparse.scores[step].float(), dense.scores[step].float()
        assert torch.isfinite(got).all()
        assert float((got - want).abs().max()) <= 6e-2, (step, float((got - want).abs().max()))
    assert torch.equal(sparse.sequences[:, : prompt_length + 2], dense.sequences[:, : prompt_length + 2]) or \
        float((dense.scores[1].float().topk(2).values.diff().abs())) < 6e-2
    for step in range(2, new_tokens):
        assert torch.isfinite(sparse.scores[step].float()).all()
    assert sparse.sequences.shape == (1, prompt_length + new_tokens)
