"""The engine once at real layer sizes: the layers of Llama 3.2 1B (width 2,048, 32 heads on 8 kv
heads of 64, feed-forward 8,192, vocabulary 128,256, llama3 rotation with factor 32 over 8,192
original positions, tied output matrix), 2 of its 16 layers, random weights. Three requests run
whole, as a prompt followed by single tokens, and mixed with each other on a pool so small that
pages are used again, in 32-bit and in bfloat16, against the plain implementation on the CPU.
The tiny configurations cannot show a fault that needs these sizes: a product over 8,192 values,
a row of 128,256 logits, the bands of the llama3 rule at this factor."""
import numpy as np
import pytest
import torch

import replay
import tiny

pytestmark = pytest.mark.gpu

LAYERS_RUN, LAYERS_FULL = 2, 16
CFG_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 2048, "num_hidden_layers": LAYERS_RUN, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
    "max_position_embeddings": 131072, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}
LENGTHS = [40, 300, 700]
TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}     # per position; measured 5.5e-6 and 1.2e-2


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    from rllm_b200.weights import write_random_model
    d = str(tmp_path_factory.mktemp("real") / "llama_1b_2_of_16_layers")
    write_random_model(CFG_1B, 5, d, std=0.02, norm_std=0.1, dtype=torch.bfloat16)
    reqs = {f"r{i}": tiny.random_prompt(n, CFG_1B["vocab_size"], 200 + i) for i, n in enumerate(LENGTHS)}
    return d, reqs, replay.plain_logits(d, reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", ["whole", "prefill_then_decode", "mixed"])
def test_two_of_sixteen_layers_at_1b_sizes(setup, dtype, family):
    from rllm_b200.engine import load_engine
    d, reqs, plain = setup
    make = {"whole": replay.whole, "prefill_then_decode": replay.prefill_then_decode,
            "mixed": lambda r: replay.mixed(r, max_live=3, chunk_sizes=(130, 64, 9, 200, 2), decode_tail=32)}[family]
    steps = make(reqs)
    eng = load_engine(d, dtype=dtype, page_size=16, max_tokens=replay.max_live_tokens(steps, reqs), max_requests=4)
    got = replay.run_in_process(eng, steps)
    worst = replay.compare(got, plain, TOL[dtype], f"1B sizes, {LAYERS_RUN} of {LAYERS_FULL} layers, {dtype} {family}",
                           per_position=True)
    assert all(n == eng.cache.groups[0].pool.num_pages for n in eng.cache.free_pages())
    # greedy tokens: where the plain logits' best two are further apart than the error allows, the
    # engine picks the same token
    agree = total = 0
    for key, row in plain.items():
        top2 = np.partition(row, -2)[-2:]
        if top2[1] - top2[0] > 2 * TOL[dtype] * float(np.abs(row).max()):
            total += 1
            agree += int(np.argmax(got[key]) == np.argmax(row))
    assert agree == total and total > 0
    print(f"1B sizes {dtype} {family}: worst relative error {worst:.2e}; {agree}/{total} decided greedy tokens agree")
