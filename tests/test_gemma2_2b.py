"""The whole Gemma-2 2B model (26 layers, 256,000-row vocabulary, window 4,096) with seeded random weights:
32-bit and bfloat16 logits against the plain implementation under each way of cutting the work.  One folder of
5 GB is written to a temporary place and read by both sides; the plain implementation works in 64 bits on the
host (about 21 GB of memory), so the test is skipped on a host with less than 48 GB free."""
import pytest
import torch

import plain_gemma2 as plain
import replay
from tolerances import SPLITS, VS_PLAIN, rel_err

pytestmark = pytest.mark.gpu

GEMMA2_2B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 26, "hidden_size": 2304, "num_attention_heads": 8, "num_key_value_heads": 4,
    "head_dim": 256, "intermediate_size": 9216, "vocab_size": 256000, "rope_theta": 10000.0,
    "sliding_window": 4096, "query_pre_attn_scalar": 256, "attn_logit_softcapping": 50.0,
    "final_logit_softcapping": 30.0, "max_position_embeddings": 8192, "rms_norm_eps": 1e-6,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "eos_token_id": 1, "torch_dtype": "bfloat16",
}


@pytest.fixture(scope="module")
def model_2b(tmp_path_factory):
    import psutil
    if psutil.virtual_memory().available < 48 * 2 ** 30:
        pytest.skip("the plain implementation of the whole 2B model needs about 21 GB of host memory")
    from tiny import make_folder
    folder = make_folder(GEMMA2_2B, seed=2, store_dtype="bfloat16", root=tmp_path_factory.mktemp("gemma2_2b"),
                         device="cuda:0")                        # (2.6 billion values: drawn on the GPU)
    cfg, w = plain.read_model_folder(folder)
    reqs = [replay.random_ids(cfg["vocab_size"], n, 600 + n) for n in (40, 9, 70)]
    ref = [plain.logits(cfg, w, r) for r in reqs]
    del w
    return {"folder": folder, "reqs": reqs, "ref": ref}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_2b_model_against_the_plain_implementation(model_2b, dtype):
    from airframe_b200.engine import GpuRuntime
    rt = GpuRuntime.load(model_2b["folder"], dtype=dtype, max_tokens=64 * 8, max_sequences=4)
    reqs, ref = model_2b["reqs"], model_2b["ref"]
    whole = [replay.run_whole(rt, r) for r in reqs]
    for got, want in zip(whole, ref):
        assert got.shape == want.shape == (len(got), 256000)
        assert rel_err(got, want) < VS_PLAIN[dtype]
    for r, w_, want in zip(reqs, whole, ref):                    # the last tokens one by one
        tail = replay.run_tail(rt, r, 8)
        assert rel_err(tail, want) < VS_PLAIN[dtype] and rel_err(tail, w_) < SPLITS[dtype]
    got, _ = replay.run_batches(rt, reqs, 3, [20, 9, 33])        # unequal prompts in one step, then single tokens
    for i, want in enumerate(ref):
        assert rel_err(got[i], want) < VS_PLAIN[dtype] and rel_err(got[i], whole[i]) < SPLITS[dtype]
    if dtype == "float32":
        # greedy tokens: the same as the plain implementation's wherever its own margin is clear
        top2 = torch.cat(ref).topk(2, -1).values
        clear = (top2[:, 0] - top2[:, 1]) > 10 * VS_PLAIN[dtype] * torch.cat(ref).abs().max()
        assert bool((torch.cat(whole).argmax(-1)[clear] == torch.cat(ref).argmax(-1)[clear]).all())
        assert int(clear.sum()) > 0
    del rt
    torch.cuda.empty_cache()
