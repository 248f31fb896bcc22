"""Shared by the tests: the two tiny Gemma 2 configurations, model folders
with random weights in a temporary place, and the oracle's view of them."""
from __future__ import annotations

import json
import os

import torch

import brolm_b200 as bb

# Tiny configurations that differ in every size and option.  A and B are the two that the benchmark
# description states (B: multi-query, a score scale that is not head_dim ** -0.5, prompts beyond the
# window); C is B with a vocabulary and a feed-forward width that are no multiples of 8 or of a tile.
TINY_A = dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, rope_theta=10000.0, sliding_window=8,
              attn_logit_softcapping=50.0, final_logit_softcapping=30.0, query_pre_attn_scalar=16,
              rms_norm_eps=1e-6, max_position_embeddings=64)
TINY_B = dict(vocab_size=512, hidden_size=96, intermediate_size=320, num_hidden_layers=3, num_attention_heads=6,
              num_key_value_heads=1, head_dim=32, rope_theta=1000.0, sliding_window=16,
              attn_logit_softcapping=20.0, final_logit_softcapping=15.0, query_pre_attn_scalar=24,
              rms_norm_eps=1e-5, max_position_embeddings=128)
TINY_C = dict(TINY_B, vocab_size=500, intermediate_size=328)
TINY = {"A": (TINY_A, 0, 0.02), "B": (TINY_B, 1, 0.05), "C": (TINY_C, 2, 0.05)}     # name -> (config, seed, weight std)


def make_folder(tmp_path, name: str, store=torch.float32) -> str:
    cfg_dict, seed, std = TINY[name]
    folder = os.path.join(str(tmp_path), f"tiny_{name}_{str(store).split('.')[-1]}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        bb.write_random_model(bb.Gemma2Config(**cfg_dict), folder, seed=seed, weight_std=std, norm_std=0.1,
                              dtype=store)
    return folder


def oracle_inputs(folder: str):
    """(config dict, {name: tensor}) read without the framework's own reader."""
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as fh:
        config = json.load(fh)
    return config, load_file(os.path.join(folder, "model.safetensors"))


def random_prompts(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
