"""Makes tests/golden/*: logits of wenhaoli-xmu/ReTurn's own Qwen3 path on two tiny random models.

Run once on a CPU box that has the reference checkout, triton and torch:

    python tests/golden/make_golden.py /path/to/ReTurn

What runs is the reference's code: its replaced forwards (rollout/monkey_patch/qwen3.py), its
Triton attention and norm kernels under TRITON_INTERPRET=1, its KV cache and its
``Model.prefill`` / ``Model.decode``.  What does not: the reference keeps a Hugging Face model as
a container for weights; this script gives it a container of its own (the attribute names the
reference touches, nothing more), so no library model code takes part.  ``scaling`` and
``inv_freq`` follow the reference's own fallbacks (rollout/attention.py:195;
rollout/utils/test_decode.py:14-17).  The reference's pools and rope tables are bfloat16; they
are replaced by float32 ones here, so that the logits are the reference's formulas in 32-bit.

Output per case: ``<case>/config.json``, ``<case>/model.safetensors`` (the weights the reference
ran with) and ``<case>/golden.json`` (prompts, page size, chunk, and the recorded logits rows).
"""
import contextlib
import json
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py PATH_TO_THE_REFERENCE_CHECKOUT")
REF = sys.argv[1]
sys.path.insert(0, REF)

import torch
from torch import nn

torch.Tensor.pin_memory = lambda self, *a, **k: self          # no CUDA on this box
torch.cuda.device = lambda dev: contextlib.nullcontext()

import rollout.constant as rconst
import rollout.cache as rcache
import rollout.model as rmodel
import rollout.monkey_patch.qwen3 as rq3

from return_b200.config.model_config import Qwen3Config
from return_b200.weights import loader
from return_b200.weights.safetensors_io import ModelFiles

rmodel._pick_num_splits = lambda n, kvh, dev, ns_max=64: 2


class Qwen3RMSNorm(nn.Module):                # the class name is what the reference's patch looks for
    def __init__(self, n, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(n))
        self.variance_epsilon = eps


class _Attn(nn.Module):
    def __init__(self, c):
        super().__init__()
        H, D = c.hidden_size, c.head_dim
        self.head_dim, self.scaling, self.sliding_window = D, D ** -0.5, None
        self.q_proj = nn.Linear(H, c.num_attention_heads * D, bias=False)
        self.k_proj = nn.Linear(H, c.num_key_value_heads * D, bias=False)
        self.v_proj = nn.Linear(H, c.num_key_value_heads * D, bias=False)
        self.o_proj = nn.Linear(c.num_attention_heads * D, H, bias=False)
        self.q_norm, self.k_norm = Qwen3RMSNorm(D, c.rms_norm_eps), Qwen3RMSNorm(D, c.rms_norm_eps)


class _MLP(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.gate_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.up_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.down_proj = nn.Linear(c.intermediate_size, c.hidden_size, bias=False)


class _Layer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.self_attn, self.mlp = _Attn(c), _MLP(c)
        self.input_layernorm = Qwen3RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.post_attention_layernorm = Qwen3RMSNorm(c.hidden_size, c.rms_norm_eps)


class _Rotary(nn.Module):
    def __init__(self, c):
        super().__init__()
        half = c.head_dim // 2
        self.inv_freq = 1.0 / (c.rope_theta ** (torch.arange(0, half).float() / half))
        self.attention_scaling = 1.0


class _Inner(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size)
        self.layers = nn.ModuleList([_Layer(c) for _ in range(c.num_hidden_layers)])
        self.norm = Qwen3RMSNorm(c.hidden_size, c.rms_norm_eps)
        self.rotary_emb = _Rotary(c)


class Container(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.config = c
        self.model = _Inner(c)
        self.lm_head = nn.Linear(c.hidden_size, c.vocab_size, bias=False)


class FakeReq:                                   # after rollout/utils/check_correctness.py:10-19
    temperature, top_p, top_k = 0.0, 1.0, 0
    subs, swap = (), ()
    ephem_at = swap_at = None
    max_new_tokens = 8

    def __init__(self, rid, ids):
        self.id, self.prompt_ids, self.split_ids, self.output = rid, list(ids), [], []

    @property
    def last_token(self):
        return self.output[-1]


def run_case(name, cfg, seed, prompt_lens, ids_seed, page, chunk, decode_steps):
    out_dir = os.path.join(HERE, name)
    loader.write_random_model(out_dir, cfg, seed, torch.float32)
    files = ModelFiles(out_dir)
    sd = {n: files.tensor(n) for n in files.names()}
    if cfg.tie_word_embeddings:
        sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
    box = Container(cfg).float().eval()
    missing, unexpected = box.load_state_dict(sd, strict=False)
    assert not missing and not unexpected, (missing, unexpected)

    rconst.PAGE_SIZE = rcache.PAGE_SIZE = rq3.PAGE_SIZE = page
    rmodel.PREFILL_CHUNK = chunk
    n_pages = 64
    m = rq3.QwenModel(box, max_token=page * n_pages, max_reside=4, device="cpu")
    kv = m.kv
    kv.k_pool = [t.float() for t in kv.k_pool]
    kv.v_pool = [t.float() for t in kv.v_pool]
    kv.k_flat = [t.view(-1, kv.num_kv_heads, kv.head_dim) for t in kv.k_pool]
    kv.v_flat = [t.view(-1, kv.num_kv_heads, kv.head_dim) for t in kv.v_pool]
    inner = m.model.model
    fr = torch.outer(torch.arange(page * (n_pages + 1)).float(), inner.rotary_emb.inv_freq.float())
    inner._rope_cos, inner._rope_sin = fr.cos().contiguous(), fr.sin().contiguous()

    records = []
    orig = rmodel.sample

    def recording_sample(logits, reqs):
        toks = orig(logits, reqs)
        for r, row in zip(reqs, logits):
            # the row is the logits after the request's len(prompt)+len(output) tokens so far
            records.append({"request": r.id, "position": len(r.prompt_ids) + len(r.output) - 1,
                            "logits": [float(x) for x in row.detach().float()]})
        return toks

    rmodel.sample = recording_sample
    g = torch.Generator().manual_seed(ids_seed)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in prompt_lens]
    reqs = [FakeReq(i, p) for i, p in enumerate(prompts)]
    for r in reqs:
        kv.alloc(r.id)
    for r, t in zip(reqs, m.prefill(reqs)):
        r.output.append(t)
    for _ in range(decode_steps):
        for r, t in zip(reqs, m.decode(reqs)):
            r.output.append(t)
    rmodel.sample = orig
    with open(os.path.join(out_dir, "golden.json"), "w") as f:
        json.dump({"page_size": page, "prefill_chunk": chunk, "prompts": prompts,
                   "outputs": [r.output for r in reqs], "records": records}, f)
    print(name, "outputs", [r.output for r in reqs], "records", len(records))


if __name__ == "__main__":
    case_a = Qwen3Config.from_dict(dict(
        vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, rope_theta=10000.0, rms_norm_eps=1e-6,
        tie_word_embeddings=True, max_position_embeddings=128))
    case_b = Qwen3Config.from_dict(dict(
        vocab_size=80, hidden_size=40, intermediate_size=56, num_hidden_layers=2, num_attention_heads=3,
        num_key_value_heads=1, head_dim=32, rope_theta=1000000.0, rms_norm_eps=1e-5,
        tie_word_embeddings=False, max_position_embeddings=256))
    run_case("ref_case_a", case_a, seed=0, prompt_lens=(5, 17, 33), ids_seed=1, page=16, chunk=8192, decode_steps=3)
    run_case("ref_case_b", case_b, seed=2, prompt_lens=(1, 9, 40), ids_seed=3, page=8, chunk=13, decode_steps=2)
