#!/usr/bin/env python3
"""Makes the golden outputs that anchor ``tests/plain_qwen2.py`` on the reference's own model code.

Run once, on the CPU, with the reference checkout importable:

    python tests/golden/make_reference_golden.py /path/to/reference/src

It imports ``mini_llm_runtime`` from that path (pure torch on the CPU; the CUDA extension there is
only built on first kernel call and is never touched here), builds
* tiny configuration A (tied head): the reference's ``QwenPrefillRunner.prefill`` gives the logits of
  every position of a 33-token prompt and the hidden state after every layer;
* tiny configuration B (untied head, which the reference's config class rejects): the reference's
  ``_decoder_layer`` function is called layer by layer on B's weights, giving the hidden state
  after every layer; the logits are the reference's ``_rms_norm`` of the last hidden state times
  ``lm_head.weight`` (the one product the reference does not have: it always multiplies by the
  embedding, qwen_model_runner.py:289-290);
* tiny configuration D (a sliding window on the layers from ``max_window_layers`` on, which the
  reference never reads): the reference's ``_decoder_layer`` with its ``packed_causal_mask``
  argument, given a mask that lets position p see the keys p-window+1 .. p on the windowed
  layers and 0 .. p on the others; logits through the tied head as the reference computes them.
  So the arithmetic of a windowed layer is the reference's own; only the rule which keys a window
  hides, and which layers have one, is this repository's reading of the config.json keys.
Weights come from this repository's seeded random-weights mode (seed 5, float32), the prompt from
``harness.random_prompt``.  The outputs are stored next to this script as float32 ``.npy`` files;
``tests/test_plain.py`` compares the plain implementation with them without needing the reference.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from harness import random_prompt  # noqa: E402
from mini_llm_runtime_b200.models import build_model  # noqa: E402
from mini_llm_runtime_b200.weights import random_tensors  # noqa: E402
from tiny_configs import TINY_A, TINY_B, TINY_D  # noqa: E402

SEED = 5


def tensors_for(config):
    model = build_model(config, torch.float32)
    return random_tensors(model.expected_tensors(), SEED, torch.float32)


def main() -> None:
    sys.path.insert(0, sys.argv[1])
    from mini_llm_runtime.qwen_config import QwenConfig
    from mini_llm_runtime.qwen_model_runner import QwenPrefillRunner, _decoder_layer, _rms_norm
    from mini_llm_runtime.qwen_weights import QwenWeights

    # ---- A: whole model through the reference's runner
    keys = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "max_position_embeddings", "rms_norm_eps", "rope_theta", "hidden_act",
            "tie_word_embeddings")
    config_a = QwenConfig(**{k: getattr(TINY_A, k) for k in keys})
    tensors_a = tensors_for(TINY_A)
    runner = QwenPrefillRunner(config_a, QwenWeights.from_state_dict(config_a, tensors_a))
    prompt_a = random_prompt(TINY_A.vocab_size, 33, 300)
    output = runner.prefill(torch.tensor([prompt_a]), return_layer_outputs=True)
    np.save(os.path.join(HERE, "tiny_a_logits.npy"), output.logits[0].numpy().astype(np.float32))
    np.save(os.path.join(HERE, "tiny_a_layers.npy"),
            torch.stack([layer[0] for layer in output.layer_outputs]).numpy().astype(np.float32))

    # ---- B: decoder stack through the reference's layer function (tied flag forced to pass its check)
    values = {k: getattr(TINY_B, k) for k in keys}
    values["tie_word_embeddings"] = True
    config_b = QwenConfig(**values)
    tensors_b = tensors_for(TINY_B)
    tied_view = {k: v for k, v in tensors_b.items() if k != "lm_head.weight"}
    weights_b = QwenWeights.from_state_dict(config_b, tied_view)
    prompt_b = random_prompt(TINY_B.vocab_size, 40, 301)
    ids = torch.tensor([prompt_b])
    x = torch.nn.functional.embedding(ids, weights_b.embedding)
    positions = torch.arange(len(prompt_b)).unsqueeze(0)
    layers = []
    with torch.inference_mode():
        for layer in weights_b.layers:
            x = _decoder_layer(x, positions, layer, config_b, apply_causal_mask=True)
            layers.append(x[0].clone())
    np.save(os.path.join(HERE, "tiny_b_layers.npy"), torch.stack(layers).numpy().astype(np.float32))
    with torch.inference_mode():
        normed = _rms_norm(x, weights_b.final_norm, config_b.rms_norm_eps)
        logits_b = torch.nn.functional.linear(normed, tensors_b["lm_head.weight"])[0]
    np.save(os.path.join(HERE, "tiny_b_logits.npy"), logits_b.numpy().astype(np.float32))

    # ---- D: windowed layers through the reference's layer function and its mask argument
    assert TINY_D.head_dim == TINY_D.hidden_size // TINY_D.num_attention_heads   # the reference derives it
    config_d = QwenConfig(**{k: getattr(TINY_D, k) for k in keys})
    tensors_d = tensors_for(TINY_D)
    weights_d = QwenWeights.from_state_dict(config_d, tensors_d)
    prompt_d = random_prompt(TINY_D.vocab_size, 150, 302)
    ids = torch.tensor([prompt_d])
    x = torch.nn.functional.embedding(ids, weights_d.embedding)
    positions = torch.arange(len(prompt_d)).unsqueeze(0)
    query, key = positions[0].unsqueeze(1), positions[0].unsqueeze(0)
    causal = key <= query
    windowed = causal & (key > query - TINY_D.sliding_window)
    layers = []
    with torch.inference_mode():
        for index, layer in enumerate(weights_d.layers):
            has_window = TINY_D.use_sliding_window and index >= TINY_D.max_window_layers
            x = _decoder_layer(x, positions, layer, config_d, apply_causal_mask=False,
                               packed_causal_mask=windowed if has_window else causal)
            layers.append(x[0].clone())
        normed = _rms_norm(x, weights_d.final_norm, config_d.rms_norm_eps)
        logits_d = torch.nn.functional.linear(normed, weights_d.embedding)[0]
    # positions 100..149 only (all past the window of 70, so the window decides what they see)
    np.save(os.path.join(HERE, "tiny_d_layers.npy"), torch.stack(layers)[:, 100:].numpy().astype(np.float32))
    np.save(os.path.join(HERE, "tiny_d_logits.npy"), logits_d[-8:].numpy().astype(np.float32))
    print("golden files written to", HERE)


if __name__ == "__main__":
    main()
