"""Grammar-constrained output: masks, state walk, verify rows, and an end-to-end constrained generation on CPU."""
import json

import pytest
import torch

xgr = pytest.importorskip("xgrammar")

from hibana_b200.engine import grammar as G                                   # noqa: E402

EOS = 257


def _grammars():
    vocab = [bytes([i]) for i in range(256)] + [b"<bos>", b"<eos>", b"<pad>"]
    return G.Grammars(vocab, vocab_size=259, stop_ids=[EOS])


def _allowed(mask, tok):
    return bool((int(mask[tok >> 5]) >> (tok & 31)) & 1)


def test_mask_follows_grammar_and_completes():
    gs = _grammars()
    st = gs.state(gs.regex(r"ab+c"))
    m = st.mask()
    assert _allowed(m, ord("a")) and not _allowed(m, ord("b")) and not _allowed(m, EOS)
    for ch in "abb":
        st.push(ord(ch))
    m = st.mask()
    assert _allowed(m, ord("b")) and _allowed(m, ord("c")) and not _allowed(m, ord("a"))
    st.push(ord("c"))
    m = st.mask()
    assert m is None or (_allowed(m, EOS) and not _allowed(m, ord("c")))
    st.push(EOS)
    assert st.complete and st.mask() is None


def test_json_schema_and_cache():
    gs = _grammars()
    schema = {"type": "object", "properties": {"n": {"type": "integer"}}, "required": ["n"]}
    c1, c2 = gs.json_schema(schema), gs.json_schema(json.dumps(schema))
    assert c1.compiled is c2.compiled and c1.kind == "json_schema"
    st = gs.state(c1)
    for ch in '{"n": 12}':
        assert _allowed(st.mask(), ord(ch)), ch
        st.push(ord(ch))
    assert not st.failed
    assert gs.recompile(c1.kind, c1.source).compiled is c1.compiled


def test_think_block_is_free():
    gs = _grammars()
    st = gs.state(gs.regex(r"yes|no", think_end=ord(">")))
    assert st.mask() is None                     # reasoning: anything goes
    for ch in "hm":
        st.push(ord(ch))
    st.push(ord(">"))
    m = st.mask()
    assert _allowed(m, ord("y")) and _allowed(m, ord("n")) and not _allowed(m, ord("h"))


def test_verify_masks_rolls_back():
    gs = _grammars()
    st = gs.state(gs.regex(r"abc"))
    rows = st.verify_masks([ord("a"), ord("x"), ord("c")])
    assert len(rows) == 4
    assert _allowed(rows[0], ord("a")) and _allowed(rows[1], ord("b")) and not _allowed(rows[1], ord("x"))
    assert rows[2] is None and rows[3] is None            # past the refused token
    assert _allowed(st.mask(), ord("a"))                  # the state did not move
    stacked = G.stack_masks(rows, gs.words)
    assert stacked.shape == (4, gs.words) and int(stacked[2, 0]) == -1


def test_constrained_generation_end_to_end_cpu():
    """A random-init model can only produce text of the grammar; unconstrained requests in the same batch are free."""
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny, scaled

    t = scaled(dense_tiny(), weight_format="bf16", vocab=259)
    model = DenseModel(t, "cpu", seed=0)
    gs = _grammars()
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"],
              "additionalProperties": False}
    sp = [SamplingParams(max_tokens=40, constraint=gs.json_schema(schema), stop_ids=(EOS,)),
          SamplingParams(max_tokens=12),
          SamplingParams(max_tokens=40, temperature=0.9, seed=5, constraint=gs.regex(r"(ab|cd){2,4}!"),
                         stop_ids=(EOS,))]
    ex = Executor(model, max_batch=4, max_ctx=128, use_graphs=False)
    prompts = [list(b"json please"), list(b"free text"), list(b"pattern")]      # token i = byte i in this vocab
    out = ex.generate_batch(prompts, sp)
    text0 = bytes(i for i in out[0].output_ids if i < 256).decode()
    assert json.loads(text0) in ({"ok": True}, {"ok": False}) and out[0].finish_reason == "stop"
    import re
    text2 = bytes(i for i in out[2].output_ids if i < 256).decode()
    assert re.fullmatch(r"(ab|cd){2,4}!", text2), text2
    assert len(out[1].output_ids) == 12 and out[1].grammar is None


def test_constrained_output_with_speculation_matches_plain_cpu():
    """Drafts are walked through the grammar (verify_masks): constrained greedy output is the same with and without
    speculative decoding, and always inside the grammar."""
    import re
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny, scaled

    t = scaled(dense_tiny(), weight_format="bf16", vocab=259)
    model = DenseModel(t, "cpu", seed=0)
    gs = _grammars()
    pat = r"((ab|cd)x){3,6}!"
    sp = [SamplingParams(max_tokens=40, constraint=gs.regex(pat), stop_ids=(EOS,)), SamplingParams(max_tokens=10)]
    prompts = [list(b"abxabxabx repeat"), list(b"free")]
    plain = Executor(model, max_batch=4, max_ctx=128, use_graphs=False).generate_batch(prompts, sp)
    ex = Executor(model, max_batch=4, max_ctx=128, use_graphs=False)
    ex.enable_spec(depth=4, proposer="ngram")
    spec = ex.generate_batch(prompts, sp)
    assert [r.output_ids for r in spec] == [r.output_ids for r in plain]
    text = bytes(i for i in spec[0].output_ids if i < 256).decode()
    assert re.fullmatch(pat, text), text
    assert not spec[0].grammar.failed


@pytest.mark.gpu
def test_constrained_generation_gpu_graphs_and_speculation():
    """The grammar bitmask is read by the sampling kernels inside the captured decode graph; with a proposer the
    verify rows are masked too. Output stays inside the grammar, unconstrained neighbours are untouched."""
    import re
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import SamplingParams
    from hibana_b200.models.dense import DenseModel
    from hibana_b200.target import dense_tiny, scaled

    t = scaled(dense_tiny(), weight_format="bf16", vocab=259)
    model = DenseModel(t, "cuda", seed=0, init_device="cpu")
    gs = _grammars()
    pat = r"((ab|cd)x){3,6}!"
    sp = [SamplingParams(max_tokens=40, constraint=gs.regex(pat), stop_ids=(EOS,)), SamplingParams(max_tokens=10),
          SamplingParams(max_tokens=40, temperature=0.8, seed=3, constraint=gs.regex(pat), stop_ids=(EOS,))]
    prompts = [list(b"abxabxabx repeat"), list(b"free"), list(b"sampled")]
    ex = Executor(model, max_batch=4, max_ctx=128, use_graphs=True)
    ex.capture_graphs()
    out = ex.generate_batch(prompts, sp)
    for i in (0, 2):
        text = bytes(x for x in out[i].output_ids if x < 256).decode()
        assert re.fullmatch(pat, text), text
    free_alone = Executor(model, max_batch=4, max_ctx=128, use_graphs=True)
    free_alone.capture_graphs()
    assert free_alone.generate_batch(prompts[1:2], sp[1:2])[0].output_ids == out[1].output_ids
    ex2 = Executor(model, max_batch=4, max_ctx=128, use_graphs=False)
    ex2.enable_spec(depth=4, proposer="ngram")
    spec = ex2.generate_batch(prompts[:2], sp[:2])
    assert spec[0].output_ids == out[0].output_ids and spec[1].output_ids == out[1].output_ids
