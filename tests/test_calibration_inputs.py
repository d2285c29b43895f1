"""Calibration-sample pipeline: seeded per-source draw with the evaluation filter, resumable generation, packing."""
import json

from hibana_b200.weights import calibration_inputs as ci


def _long(i):
    return " ".join(f"word{i}x{j}" for j in range(20))


def test_prompt_draw_is_equal_per_source_seeded_and_drops_evaluation_items(tmp_path):
    chat = tmp_path / "chat.jsonl"
    chat.write_text("\n".join(json.dumps({"messages": [{"role": "system", "content": "s"},
                                                        {"role": "user", "content": f"Please explain topic {i}. " + _long(i)},
                                                        {"role": "assistant", "content": "never read"}]})
                              for i in range(30)))
    code = tmp_path / "code.txt"
    code.write_text("\n\n".join(f"Write a function number {i}" for i in range(10)) + "\n\nWhat is 2 + 2?")
    evals = tmp_path / "evals"
    evals.mkdir()
    # evaluation items: one shares a 13-word span with chat prompt 3, one equals a short code prompt
    (evals / "a.jsonl").write_text(json.dumps({"question": "Intro. " + _long(3) + " and more", "answer": "x"}) + "\n")
    (evals / "b.tsv").write_text("what is 2 + 2?\t4\n")
    args = ["prompts", "--sources", str(chat), str(code), "--evals", str(evals), "--per-source", "8", "--seed", "1",
            "--output", str(tmp_path / "p.json")]
    ci.main(args)
    doc = json.loads((tmp_path / "p.json").read_text())
    by = {}
    for p in doc["prompts"]:
        by.setdefault(p["source"], []).append(p["prompt"])
    assert {k: len(v) for k, v in by.items()} == {"chat": 8, "code": 8}
    assert doc["sources"] == {"chat": 30, "code": 11}
    every = ci.draw({"chat": ci.load_prompts(chat), "code": ci.load_prompts(code)}, 100, 1,
                    ci.EvalFilter.from_directory(evals))
    texts = [p["prompt"] for p in every]
    assert len(texts) == 29 + 10                       # chat prompt 3 and "What is 2 + 2?" are evaluation items
    assert not any("topic 3." in t for t in texts) and "What is 2 + 2?" not in texts
    assert all("never read" not in t for t in texts)
    ci.main(args[:-1] + [str(tmp_path / "p2.json")])
    assert json.loads((tmp_path / "p2.json").read_text())["prompts"] == doc["prompts"]     # same seed, same draw


def test_generation_resumes_and_build_packs_whole_turns(tmp_path):
    from hibana_b200.api.chat_template import ChatTemplate
    from hibana_b200.tokenizer import ByteTokenizer
    prompts = [{"source": "s", "prompt": f"question {i}"} for i in range(6)]
    calls = []

    def ask(p, fail_after=None):
        calls.append(p)
        if fail_after is not None and len(calls) > fail_after:
            raise RuntimeError("server went away")
        return {"reasoning": f"thinking about {p}", "answer": f"answer to {p} " * (40 if p.endswith("4") else 2)}
    out = tmp_path / "answers.json"
    try:
        ci.generate(prompts, out, lambda p: ask(p, fail_after=3), concurrency=1)
    except RuntimeError:
        pass
    assert len((tmp_path / "answers.json.partial.jsonl").read_text().splitlines()) == 3
    calls.clear()
    answers = ci.generate(prompts, out, ask, concurrency=2)
    assert sorted(calls) == ["question 3", "question 4", "question 5"]      # the finished ones were not asked again
    assert [a["prompt"] for a in answers] == [p["prompt"] for p in prompts]
    tok, tpl = ByteTokenizer(), ChatTemplate()
    samples = ci.build(answers, tpl, tok, max_tokens=400)
    turns = [tok.encode(ci.render_turn(tpl, a["prompt"], a["reasoning"], a["answer"])) for a in answers]
    assert "<think>" in ci.render_turn(tpl, "q", "r", "a") and "<think>" not in ci.render_turn(tpl, "q", "", "a")
    assert all(len(s) <= 400 for s in samples)
    assert max(len(t) for t in turns) > 400                                  # the long turn was cut
    flat = [x for s in samples for x in s]
    assert flat == [x for t in turns for x in t[:400]]                       # whole turns, in order, nothing else
    # every sample boundary falls between two turns
    ends, n = set(), 0
    for t in turns:
        n += min(len(t), 400)
        ends.add(n)
    n = 0
    for s in samples:
        n += len(s)
        assert n in ends
    (tmp_path / "a.json").write_text(json.dumps({"answers": answers}))
    ci.main(["build", "--target", "dense-tiny", "--answers", str(tmp_path / "a.json"), "--max-tokens", "400",
             "--output", str(tmp_path / "samples.json")])
    from hibana_b200.weights.calibrate_model import load_samples
    assert load_samples(tmp_path / "samples.json") == samples
