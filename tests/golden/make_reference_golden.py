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
  after every layer; the untied head has no counterpart and rests on its formula.
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
from tiny_configs import TINY_A, TINY_B  # noqa: E402

SEED = 5


def tensors_for(config):
    model = build_model(config, torch.float32)
    return random_tensors(model.expected_tensors(), SEED, torch.float32)


def main() -> None:
    sys.path.insert(0, sys.argv[1])
    from mini_llm_runtime.qwen_config import QwenConfig
    from mini_llm_runtime.qwen_model_runner import QwenPrefillRunner, _decoder_layer
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
    print("golden files written to", HERE)


if __name__ == "__main__":
    main()
