"""The Kilatar design through the engine against the plain implementation (tests/plain_kilatar.py): whole prompts,
token-by-token decoding, portions down to two tokens, unequal batches, pages and slots that change hands, the captured
decode step, long decoding past every chunk, and greedy generation through the entry point and the scheduler.  Small
configurations of their own (tests/kilatar_cases.py)."""
import pytest
import torch

import kilatar_cases as cases
import plain_kilatar

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompt_and_first_tokens(name, dtype):
    name = cases.variant(name, dtype)
    runner = cases.make_runner(name, dtype)
    for length, seed in ((1, 1), (2, 2), (3, 3), (75, 4)):  # the first tokens of a sequence, alone and in a prompt
        ids, want = cases.plain_logits(name, length, seed)
        got = cases.replay(runner, f"w{length}", ids, [length])
        cases.assert_close(got, want, dtype, f"{name} whole {length}")


@pytest.mark.parametrize("name", ["P", "Q"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_the_stream_after_every_layer_run(name, dtype):
    """Layer run by layer run (a looped layer counts each time): the float32 stream behind every block."""
    name = cases.variant(name, dtype)
    ids = cases.make_ids(name, 41, 5)
    w = {k: v.double() for k, v in cases.weights_for(name).items()}
    _, streams = plain_kilatar.forward(cases.CASES[name], w, ids, streams=True)
    runner = cases.make_runner(name, dtype)
    seen = []
    for block in runner.model.blocks:
        inner = block.forward

        def watched(ctx, acc, cache, inner=inner):
            inner(ctx, acc, cache)
            ctx.flush_pending()
            seen.append(acc.clone())

        block.forward = watched
    cases.replay(runner, "s", ids, [len(ids)])
    assert len(seen) == len(streams) == len(runner.model.spec.schedule)
    for i, (got, want) in enumerate(zip(seen, streams)):
        cases.assert_close(got.cpu(), want.float(), dtype, f"stream after layer run {i}")


@pytest.mark.parametrize("name", ["P", "Q", "R"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_then_token_by_token(name, dtype):
    name = cases.variant(name, dtype)
    ids, want = cases.plain_logits(name, 100, 7)
    runner = cases.make_runner(name, dtype)
    got = cases.replay(runner, "d", ids, [45] + [1] * 55)  # the decoded tokens cross the edges of every chunk
    cases.assert_close(got, want, dtype, f"{name} decode")
    got = cases.replay(runner, "t", ids[:40], [1] * 40)  # from the very first token on, in the slot just freed
    cases.assert_close(got, want[:40], dtype, f"{name} token by token")


@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page_size", [8, 16])
def test_portions_of_changing_size(name, dtype, page_size):
    name = cases.variant(name, dtype)
    ids, want = cases.plain_logits(name, 190, 9)
    runner = cases.make_runner(name, dtype, page_size=page_size)
    pattern = [7, 2, 5, 3, 16, 2, 9, 1, 4, 33, 2, 6, 17, 8, 15, 1, 2, 2, 13, 37]
    cuts = []
    while sum(cuts) < len(ids):
        cuts.append(min(pattern[len(cuts) % len(pattern)], len(ids) - sum(cuts)))
    got = cases.replay(runner, "c", ids, cuts)
    cases.assert_close(got, want, dtype, f"{name} portions")
    if dtype == "float32":  # the order of every sum depends on the position alone
        whole = cases.replay(runner, "w", ids, [len(ids)])
        assert torch.equal(got, whole)


@pytest.mark.parametrize("dtype", DTYPES)
def test_steps_of_many_tokens(dtype):
    """330 tokens in one step, and 290 behind 40 cached ones (chunks of 48 and 150 tokens inside the step and across
    its start: the second portion starts in the middle of a chunk; tensor-core products and attention in bfloat16)."""
    name = cases.variant("R", dtype)
    ids, want = cases.plain_logits(name, 330, 11)
    runner = cases.make_runner(name, dtype)
    cases.assert_close(cases.replay(runner, "a", ids, [330]), want, dtype, "330 tokens")
    cases.assert_close(cases.replay(runner, "b", ids, [40, 290]), want, dtype, "290 behind 40")


@pytest.mark.parametrize("name", ["P", "R"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_with_pages_and_slots_used_again(name, dtype):
    """Up to three live requests in three slots; the pool holds little more than the live tokens: every request later
    in the list runs in a slot and in pages that another one has left."""
    from torchlet_b200.engine import StepEntry

    name = cases.variant(name, dtype)
    lengths = (61, 23, 100, 2, 37, 48)
    seqs = [cases.plain_logits(name, n, 20 + i) for i, n in enumerate(lengths)]
    runner = cases.make_runner(name, dtype, num_pages=26, slots=3, page_size=8)
    at = [0] * len(seqs)
    got = [[] for _ in seqs]
    waiting, live = list(range(len(seqs))), []
    portions = [5, 1, 19, 2, 1, 1, 30, 3, 1, 8]
    turn = 0
    while waiting or live:
        while waiting and len(live) < 3 and runner.cache.num_free_slots:
            need = -(-lengths[waiting[0]] // 8)
            held = sum(-(-lengths[r] // 8) for r in live)
            if held + need > 25:
                break
            r = waiting.pop(0)
            runner.admit(r)
            live.append(r)
        entries, taken = [], []
        for r in live:
            size = min(portions[(turn + 3 * r) % len(portions)], lengths[r] - at[r])
            ids = seqs[r][0]
            entries.append(StepEntry(r, ids[at[r]:at[r] + size], list(range(size))))
            taken.append((r, size))
        logits = runner.step(entries).cpu()
        row = 0
        for r, size in taken:
            got[r].append(logits[row:row + size].clone())
            row += size
            at[r] += size
            if at[r] == lengths[r]:
                runner.finish(r)
                live.remove(r)
        runner.cache.check()
        turn += 1
    for r, (ids, want) in enumerate(seqs):
        cases.assert_close(torch.cat(got[r]), want, dtype, f"{name} request {r}")
    if dtype == "float32":  # each request alone gives the very same numbers
        alone = cases.replay(runner, "alone", seqs[2][0], [lengths[2]])
        assert torch.equal(torch.cat(got[2]), alone)


@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_captured_decode_step_with_padding_lanes(name, dtype):
    """Three requests decode together in a bucket of four lanes (one is padding) from the captured graph; the states of
    a fourth request, which waits meanwhile, must not be touched by the padding lane."""
    from torchlet_b200.engine import StepEntry

    lengths = (93, 72, 85, 90) if name == "R" else (33, 12, 25, 30)
    name = cases.variant(name, dtype)
    seqs = [cases.plain_logits(name, n, 40 + i) for i, n in enumerate(lengths)]
    runner = cases.make_runner(name, dtype, slots=4, cuda_graph=True)
    for r, (ids, _) in enumerate(seqs):
        runner.admit(r)
    for r, (ids, _) in enumerate(seqs):  # prompts without their last 10 tokens; request 3 stays behind
        runner.step([StepEntry(r, ids[:len(ids) - 10], [])])
    got = {r: [] for r in range(3)}
    for k in range(10):
        entries = [StepEntry(r, [seqs[r][0][len(seqs[r][0]) - 10 + k]], [0]) for r in range(3)]
        logits = runner.step(entries).cpu()
        for r in range(3):
            got[r].append(logits[r].clone())
    assert runner.graph_steps == 10
    for r in range(3):
        want = seqs[r][1][-10:]
        cases.assert_close(torch.stack(got[r]), want, dtype, f"{name} graph request {r}")
    ids, want = seqs[3]
    rest = runner.step([StepEntry(3, ids[-10:], list(range(10)))]).cpu()  # its states survived the padding lane
    cases.assert_close(rest, want[-10:], dtype, f"{name} the request that waited")


@pytest.mark.parametrize("name", ["Q", "R"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(name, dtype):
    """360 decoded tokens: chunk after chunk begins and ends among decoded tokens, passed pages are given back while
    the captured step runs, and the recurrent states and the convolution's inputs are carried 360 times."""
    name = cases.variant(name, dtype)
    ids, want = cases.plain_logits(name, 380, 78)
    runner = cases.make_runner(name, dtype, num_pages=40, cuda_graph=True)
    got = cases.replay(runner, "long", ids, [20] + [1] * 360)
    assert runner.graph_steps == 360
    cases.assert_close(got, want, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(tmp_path, dtype):
    import json

    from safetensors.torch import save_file

    from torchlet_b200 import LLM

    name = cases.variant("P", dtype)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cases.CASES[name]))
    w = cases.weights_for(name)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, str(folder / "model.safetensors"))
    llm = LLM(folder, max_decode_slots=2, kv_block_size=8, dtype=dtype, max_seq_len=96, max_num_blocks=30,
              max_num_batched_tokens=32)
    prompts = [cases.make_ids(name, n, 60 + i) for i, n in enumerate((5, 40, 17, 1))]  # more requests than slots
    new = 10
    outputs = llm.generate(prompts, max_new_tokens=new)
    assert llm.engine.runner.graph_steps > 0
    cfg, wd = cases.CASES[name], {k: v.double() for k, v in w.items()}
    for prompt, got in zip(prompts, outputs):
        assert len(got) == new
        ids = list(prompt)
        for token in got:
            logits = plain_kilatar.forward(cfg, wd, ids)[-1]
            if dtype == "float32":
                assert token == int(logits.argmax())
            else:  # bfloat16 may flip a near-tie: the token must be within rounding of the best
                assert logits[token] >= logits.max() - cases.TOLERANCE[dtype] * logits.abs().max()
            ids.append(token)
    llm.engine.runner.cache.check()
    assert llm.engine.runner.cache.live_requests() == []


def test_trace_replay_chooses_the_model_by_its_configuration(tmp_path):
    import io
    import json

    import numpy as np
    from safetensors.torch import save_file

    from torchlet_b200.engine import trace

    name = "Q"
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cases.CASES[name]))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in cases.weights_for(name).items()},
              str(folder / "model.safetensors"))
    ids, want = cases.plain_logits(name, 30, 5)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:20], "want": [0, 19]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ids[20:21], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": ids[21:], "want": [8]}], "end": ["a"]}]
    out = tmp_path / "out"
    code = trace.main(["--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "64"],
                      stdin=io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), stdout=io.StringIO())
    assert code == 0
    V = cases.CASES[name]["vocab"]
    got = torch.cat([torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)) for i in range(3)])
    cases.assert_close(got, want[[0, 19, 20, 29]], "float32", "trace replay")
