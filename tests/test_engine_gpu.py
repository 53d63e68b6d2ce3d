"""Generation through the Python entry point and the command line."""
import asyncio
import json
import os
import subprocess
import sys

import pytest
import torch

import helpers
from helpers import plain

pytestmark = pytest.mark.gpu


def _engine(model_dir, dtype="float32", **kw):
    from return_b200.engine.config import EngineConfig
    from return_b200.engine.engine import Engine
    base = dict(max_token=1024, max_reside=4, page_size=16, prefill_chunk=64, dtype=dtype, use_cuda_graph=False)
    base.update(kw)
    return Engine(model_dir, EngineConfig(**base))


def _plain_greedy(model_dir, prompts, n, stop_ids=()):
    c, w = plain.read_config(model_dir), plain.read_weights(model_dir)
    return [plain.greedy_generate(c, w, p, n, stop_ids) for p in prompts]


@pytest.mark.parametrize("case,lens,new,chunk", [("A", (5, 17, 33), 8, 64), ("B", (1, 9, 40, 71), 12, 13), ("C", (3, 50, 90), 10, 32)])
def test_greedy_generation_equals_plain(tmp_path, case, lens, new, chunk):
    d = helpers.make_model_dir(tmp_path, case)
    vocab = helpers.CASES[case][0]["vocab_size"]
    prompts = [helpers.random_ids(vocab, n, 1 + i) for i, n in enumerate(lens)]
    want = _plain_greedy(d, prompts, new)
    eng = _engine(d, "float32", page_size=helpers.CASES[case][2], prefill_chunk=chunk)
    got = eng.generate(prompts, max_new_tokens=new, temperature=0.0)
    assert [r.output_ids for r in got] == want
    assert all(r.finish_reason == "length" and r.num_tokens == new for r in got)
    # the log-probabilities are those of the raw logits
    c, w = plain.read_config(d), plain.read_weights(d)
    ids = prompts[1] + got[1].output_ids
    lg = plain.forward_logits(c, w, ids)
    for k, (tok, lp) in enumerate(zip(got[1].output_ids, got[1].output_logprobs)):
        assert abs(lp - plain.logprob(lg[len(prompts[1]) - 1 + k], tok)) < 1e-3
    assert eng.runner.manager.pages_used() == [0] * len(eng.runner.manager.groups)
    st = eng.stats()
    assert st["steps"] > 0 and st["page_used"] == 0 and st["decode_tps"] is not None


def test_bfloat16_greedy_mostly_equals_plain(tmp_path):
    d = helpers.make_model_dir(tmp_path, "B")
    prompts = [helpers.random_ids(384, n, 5 + i) for i, n in enumerate((9, 40, 71))]
    want = _plain_greedy(d, prompts, 12)
    got = _engine(d, "bfloat16", page_size=8).generate(prompts, max_new_tokens=12, temperature=0.0)
    same = sum(a == b for r, w in zip(got, want) for a, b in zip(r.output_ids, w))
    assert same >= 0.8 * 36, (same, [r.output_ids for r in got], want)
    assert [r.output_ids[0] for r in got] == [w[0] for w in want]


def test_stop_sequence(tmp_path):
    d = helpers.make_model_dir(tmp_path, "B")
    prompt = helpers.random_ids(384, 20, 3)
    free = _plain_greedy(d, [prompt], 10)[0]
    stop = [free[3:5]]
    got = _engine(d).generate([prompt], max_new_tokens=10, temperature=0.0, stop_ids=stop)[0]
    assert got.output_ids == free[:5] and got.finish_reason == "stop"
    eos = free[2]                                        # an end-of-sequence id is a stop sequence of one token
    got = _engine(d).generate([prompt], max_new_tokens=10, temperature=0.0, eos_token_id=eos)[0]
    assert got.output_ids == free[:free.index(eos) + 1] and got.finish_reason == "stop"


def test_sampling_is_reproducible_and_independent_of_the_batch(tmp_path):
    from return_b200.engine.request import Request
    d = helpers.make_model_dir(tmp_path, "B")
    prompts = [helpers.random_ids(384, n, 30 + i) for i, n in enumerate((1, 9, 40, 71))]
    mk = lambda i: Request(f"s{i}", prompts[i], max_new_tokens=12, temperature=0.8, top_p=0.95, top_k=50, seed=100 + i)
    together = _engine(d, page_size=8, prefill_chunk=13).generate([mk(i) for i in range(4)])
    again = _engine(d, page_size=8, prefill_chunk=64).generate([mk(i) for i in range(4)])
    alone = [_engine(d, page_size=8).generate([mk(i)])[0] for i in range(4)]
    for a, b, c in zip(together, again, alone):
        assert a.output_ids == b.output_ids == c.output_ids
    assert len({tuple(r.output_ids) for r in together}) == 4
    other = _engine(d, page_size=8).generate([Request("x", prompts[2], max_new_tokens=12, temperature=0.8, seed=999)])[0]
    assert other.output_ids != together[2].output_ids
    # sampled tokens lie in the kept set of the plain filter, and their log-probs are the raw ones
    c, w = plain.read_config(d), plain.read_weights(d)
    r = together[3]
    lg = plain.forward_logits(c, w, prompts[3] + r.output_ids)
    for k, tok in enumerate(r.output_ids):
        row = lg[len(prompts[3]) - 1 + k]
        assert plain.filtered_probs(row, 0.8, 50, 0.95)[tok] > 0
        assert abs(r.output_logprobs[k] - plain.logprob(row, tok)) < 1e-3


def test_pool_too_small_for_all_preempts_and_still_gives_the_same_tokens(tmp_path):
    d = helpers.make_model_dir(tmp_path, "A")
    prompts = [helpers.random_ids(256, n, 50 + i) for i, n in enumerate((30, 28, 25, 20))]
    want = _plain_greedy(d, prompts, 24)
    eng = _engine(d, max_token=160, max_reside=4, page_size=16, prefill_chunk=32)     # 10 pages for ~200 tokens
    got = eng.generate(prompts, max_new_tokens=24, temperature=0.0)
    assert [r.output_ids for r in got] == want
    assert eng.stats()["preemptions"] > 0
    eng.runner.manager.check()


def test_request_larger_than_the_pool_raises(tmp_path):
    from return_b200.cache.manager import KVCapacityError
    d = helpers.make_model_dir(tmp_path, "A")
    eng = _engine(d, max_token=64, page_size=16, max_model_len=128)
    with pytest.raises(KVCapacityError):
        eng.generate([list(range(70))], max_new_tokens=2)
    with pytest.raises(KVCapacityError):
        eng.generate([list(range(60))], max_new_tokens=10, temperature=0.0)       # outgrows the pool while decoding
    assert eng.runner.manager.pages_used() == [0] and not eng.has_unfinished()
    assert len(eng.generate([list(range(20))], max_new_tokens=4, temperature=0.0)[0].output_ids) == 4


def test_async_engine_in_the_references_shape(tmp_path):
    from return_b200.engine.engine import AsyncEngine
    from return_b200.engine.request import Request
    d = helpers.make_model_dir(tmp_path, "A")
    prompts = [helpers.random_ids(256, n, 70 + i) for i, n in enumerate((5, 17, 33))]
    want = _plain_greedy(d, prompts, 6)

    async def main():
        eng = AsyncEngine(_engine(d))
        eng.start()
        reqs = [Request(f"a{i}", p, max_new_tokens=6, temperature=0.0) for i, p in enumerate(prompts)]
        done = await asyncio.gather(*(eng.submit(r) for r in reqs))
        for r in done:
            eng.release(r.id)
        stats = eng.stats()
        await eng.stop()
        return done, stats

    done, stats = asyncio.run(main())
    assert [r.output for r in done] == want and stats["running"] == 0


def test_command_line(tmp_path):
    cfg_path = os.path.join(str(tmp_path), "config.json")
    with open(cfg_path, "w") as f:
        json.dump(helpers.tiny_config("B").to_dict(), f)
    model = os.path.join(str(tmp_path), "model")
    run = lambda *a: subprocess.run([sys.executable, "-m", "return_b200", *a], cwd=helpers.ROOT,
                                    capture_output=True, text=True, timeout=600)
    p = run("random-weights", "--config", cfg_path, "--seed", "2", "--out", model, "--dtype", "float32")
    assert p.returncode == 0, p.stderr[-2000:]
    prompt = helpers.random_ids(384, 9, 4)
    p = run("generate", "--model", model, "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
            "--new", "5", "--temperature", "0", "--max-token", "256", "--max-reside", "2", "--page-size", "8")
    assert p.returncode == 0, p.stderr[-2000:]
    out = json.loads(p.stdout.strip().splitlines()[-1])
    assert out["output_ids"] == _plain_greedy(model, [prompt], 5)[0] and out["finish_reason"] == "length"


def test_decode_that_runs_ahead_of_the_host_gives_the_same_tokens(tmp_path):
    """With captured graphs the engine launches decode step k + 1 before it has read step k's tokens.
    Requests that end at different times (by length, by a stop sequence seen one step late) and sampled
    tokens must come out as they do step by step."""
    from return_b200.engine.request import Request
    d = helpers.make_model_dir(tmp_path, "B")
    prompts = [helpers.random_ids(384, n, 21 + i) for i, n in enumerate((9, 40, 71, 5))]
    free = _plain_greedy(d, [prompts[1]], 14)[0]

    def requests():
        return [Request("a", prompts[0], max_new_tokens=5, temperature=0.7, top_p=0.9, seed=11),
                Request("b", prompts[1], max_new_tokens=14, temperature=0.0, stop_ids=[free[6:8]]),
                Request("c", prompts[2], max_new_tokens=9, temperature=1.3, top_k=20, seed=5),
                Request("d", prompts[3], max_new_tokens=20, temperature=0.0)]

    step_wise = _engine(d, page_size=8, use_cuda_graph=False).generate(requests())
    eng = _engine(d, page_size=8, use_cuda_graph=True)
    ahead = eng.generate(requests())
    assert [r.output_ids for r in ahead] == [r.output_ids for r in step_wise]
    assert [r.finish_reason for r in ahead] == ["length", "stop", "length", "length"]
    stop = free[6:8]
    first = next(i for i in range(1, 14) if free[i - 1:i + 1] == stop)     # greedy output may repeat itself
    assert ahead[1].output_ids == free[:first + 1]
    assert all(abs(x - y) < 1e-5 for r, s in zip(ahead, step_wise) for x, y in zip(r.output_logprobs, s.output_logprobs))
    assert eng.runner.manager.pages_used() == [0] * len(eng.runner.manager.groups)
    assert eng.runner.manager.free_slots == 4

    # run(max_steps) runs exactly that many steps
    eng = _engine(d, page_size=8, use_cuda_graph=True)
    reqs = [Request(f"r{i}", p, max_new_tokens=30, temperature=0.0) for i, p in enumerate(prompts)]
    for r in reqs:
        eng.add_request(r)
    while any(not r.output for r in reqs):
        eng.step()
    have, steps = [len(r.output) for r in reqs], eng.stats()["steps"]
    eng.run(max_steps=7)
    assert [len(r.output) for r in reqs] == [h + 7 for h in have] and eng.stats()["steps"] == steps + 7
    want = _plain_greedy(d, prompts, 10)
    assert [r.output[:8] for r in reqs] == [w[:8] for w in want]


def test_padded_decode_graphs_give_the_same_tokens(tmp_path):
    """Beyond 8 requests a decode step runs in the graph of the next larger batch size, the rows between
    being padding that touches no page.  Eleven requests that end one by one: same tokens as without graphs,
    few graphs, no page left behind."""
    from return_b200.engine.request import Request
    d = helpers.make_model_dir(tmp_path, "B")
    prompts = [helpers.random_ids(384, 5 + 3 * i, 90 + i) for i in range(11)]

    def requests():
        return [Request(f"p{i}", p, max_new_tokens=4 + 2 * i, temperature=0.0 if i % 2 else 0.9, top_k=30, seed=40 + i)
                for i, p in enumerate(prompts)]

    plain_steps = _engine(d, "bfloat16", page_size=8, max_reside=12, use_cuda_graph=False).generate(requests())
    eng = _engine(d, "bfloat16", page_size=8, max_reside=12, use_cuda_graph=True)
    graphed = eng.generate(requests())
    assert [r.output_ids for r in graphed] == [r.output_ids for r in plain_steps]
    sizes = sorted({n for n, _ in eng.runner._graphs})
    assert sizes and set(sizes) <= {1, 2, 3, 4, 5, 6, 7, 8, 12} and 12 in sizes, sizes
    assert [eng.runner.graph_batch_size(m) for m in (1, 8, 9, 11, 12)] == [1, 8, 12, 12, 12]          # never beyond max_reside
    assert eng.runner.capture_decode_graphs() >= 9
    assert eng.runner.manager.pages_used() == [0] * len(eng.runner.manager.groups)
    eng.runner.manager.check()


def test_running_ahead_gives_way_when_pages_run_short(tmp_path):
    """A pool too small for all: the loop that runs ahead stops, the ordinary step preempts, and the
    tokens are still those of plain greedy decoding."""
    d = helpers.make_model_dir(tmp_path, "B")
    prompts = [helpers.random_ids(384, n, 31 + i) for i, n in enumerate((30, 28, 33))]
    want = _plain_greedy(d, prompts, 24)
    eng = _engine(d, max_token=136, page_size=8, use_cuda_graph=True, max_model_len=128)
    got = eng.generate(prompts, max_new_tokens=24, temperature=0.0)
    assert [r.output_ids for r in got] == want
    assert eng.stats()["preemptions"] > 0


def test_running_ahead_with_requests_that_cross_a_page_edge_together(tmp_path):
    """Two prompts of one page each reach the page's edge in the same decode step while one page is free:
    each alone would fit, both do not.  The loop that runs ahead must see that before it takes a page, and
    leave the step to the scheduler, which preempts; the tokens stay those of plain greedy decoding."""
    d = helpers.make_model_dir(tmp_path, "A")
    prompts = [helpers.random_ids(256, 16, 61 + i) for i in range(2)]
    want = _plain_greedy(d, prompts, 20)
    eng = _engine(d, max_token=48, max_reside=2, page_size=16, use_cuda_graph=True, max_model_len=64)
    got = eng.generate(prompts, max_new_tokens=20, temperature=0.0)
    assert [r.output_ids for r in got] == want
    assert eng.stats()["preemptions"] > 0
    eng.runner.manager.check()
    assert eng.runner.manager.pages_used() == [0]


@pytest.mark.parametrize("graph", [False, True])
def test_a_kept_session_continues_in_a_second_turn(tmp_path, graph):
    """The reference keeps a session's cache when a request ends, and the next request of the session runs only
    what is new (rollout/engine.py:266-306; its check: rollout/utils/check_correctness.py:52-81, two turns).  Here
    with ``keep``: turn 1 generates, turn 2 brings the whole conversation plus new tokens; its tokens equal the
    plain implementation's on the whole context, and only the new tokens were run.  With captured graphs a stop
    sequence is seen one step late, so a token too many is in the cache and has to be taken back before keeping."""
    d = helpers.make_model_dir(tmp_path, "B")
    p1 = helpers.random_ids(384, 23, 5)
    more = helpers.random_ids(384, 11, 6)
    free = _plain_greedy(d, [p1], 10)[0]
    stop = [free[4:6]]
    first = next(i for i in range(1, 10) if free[i - 1:i + 1] == stop[0])
    eng = _engine(d, page_size=8, use_cuda_graph=graph)
    t1 = eng.generate([p1], max_new_tokens=10, temperature=0.0, stop_ids=stop, keep=True, ids=["chat"])[0]
    assert t1.output_ids == free[:first + 1] and t1.finish_reason == "stop"
    cached = len(p1) + len(t1.output_ids) - 1
    assert eng.runner.manager.length("chat") == cached and eng.stats()["kept_sessions"] == 1
    p2 = p1 + t1.output_ids + more
    want2 = _plain_greedy(d, [p2], 8)[0]
    steps_before = eng.stats()["steps"]
    t2 = eng.generate([p2], max_new_tokens=8, temperature=0.0, keep=True, ids=["chat"])[0]
    assert t2.output_ids == want2
    # the second turn's prompt went in as one portion of what was new: one step for it, then seven decode steps
    assert eng.stats()["steps"] - steps_before == 8
    assert eng.runner.manager.length("chat") == len(p2) + 7
    assert eng.release("chat") and eng.runner.manager.pages_used() == [0] and eng.runner.manager.free_slots == 4
    # without keep nothing stays
    eng.generate([p1], max_new_tokens=3, temperature=0.0, ids=["other"])
    assert eng.stats()["kept_sessions"] == 0 and eng.runner.manager.pages_used() == [0]
