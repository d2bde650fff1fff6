"""Data preparation: tokenizer, documents, the three packings, the pipeline and its reader."""
import json
from types import SimpleNamespace as NS

import numpy as np
import pytest

from bux_b200.data import packing as P
from bux_b200.data import prepared, tokenizer as TK


def test_byte_tokenizer_round_trip():
    tok = TK.ByteTokenizer(("<|endoftext|>", "<|im_start|>"))
    text = "héllo<|endoftext|>wörld<|im_start|>"
    ids = tok.encode(text)
    assert tok.decode(ids) == text
    assert ids.count(256) == 1 and ids.count(257) == 1 and tok.vocab_size == 258


def _show(rows):
    return ["".join("ABCD"[d] * n for d, _, n in row) for row in rows]


def test_the_three_packings_on_the_documented_example():
    lengths = [5, 3, 10, 2]  # A, B, C, D in rows of 8
    concat = P.plan(lengths, 8, NS(type="concat"))
    assert [sum(n for *_, n in r) for r in concat[:2]] == [8, 8]
    greedy = P.plan(lengths, 8, NS(type="greedy", long="drop", max_docs=None))
    assert _show(greedy) == ["AAAAABBB", "DD"]
    best = P.plan(lengths, 8, NS(type="best_fit", long="split", max_docs=None, sort=True))
    assert sorted(_show(best)) == sorted(["CCCCCCCC", "AAAAABBB", "CCCDD"])
    trunc = P.plan(lengths, 8, NS(type="best_fit", long="truncate", max_docs=None, sort=True))
    assert sorted(_show(trunc)) == sorted(["CCCCCCCC", "AAAAABBB", "DD"])


def test_every_token_is_a_target_once_except_document_firsts():
    rng = np.random.default_rng(0)
    lengths = rng.integers(2, 40, 50).tolist()
    docs = [np.arange(n, dtype=np.int32) + 1000 * i for i, n in enumerate(lengths)]
    masks = [np.ones(n, bool) for n in lengths]
    for pk in (NS(type="best_fit", long="split", max_docs=None, sort=True, doc_mask=True),
               NS(type="greedy", long="split", max_docs=3, doc_mask=True)):
        rows = P.plan(lengths, 16, pk)
        assert all(sum(p[2] for p in row) <= 16 for row in rows)
        ids, pos, mask = P.materialize(rows, docs, masks, 16, True)
        targets = ids[mask]
        assert len(set(targets.tolist())) == len(targets) == sum(lengths) - len(lengths)
        # positions restart at every document and at every piece
        assert (pos[:, 0] == 0).all()


def test_permutation_is_a_bijection():
    for n in (1, 2, 7, 100, 257):
        got = sorted(prepared.permuted(i, n, (3, 1)) for i in range(n))
        assert got == list(range(n))
    a = [prepared.permuted(i, 100, (3, 1)) for i in range(100)]
    b = [prepared.permuted(i, 100, (3, 2)) for i in range(100)]
    assert a != b and a != list(range(100))


def test_prepare_and_train_on_text(tmp_path):
    import torch

    from bux_b200.data import pipeline
    from bux_b200.lang import compile_runs
    from bux_b200.train.trainer import Trainer

    data = tmp_path / "docs.jsonl"
    rng = np.random.default_rng(1)
    with open(data, "w") as f:
        for i in range(200):
            words = " ".join(rng.choice(["alpha", "beta", "gamma", "delta"], rng.integers(3, 30)))
            f.write(json.dumps({"text": f"doc {i}: {words}"}) + "\n")
    src = f"""
d_model=32
vocab_size=257
n = rmsnorm
block = [n gqa(num_heads=2, num_kv_heads=1, rope=rope())] [n gated_mlp(intermediate_size=48, activation=swish)]
model = embed block^2 n head
data = text(path="{data}")
tokenizer = tokenizer(name="bytes")
optimizer = adamw(lr=1e-2)
seq_len = 64
batch = 4
steps = 8
precision = precision(compute=float32)
"""
    run = compile_runs(src, filename="t.bux")[0]
    (job,) = pipeline.jobs(run.train, tmp_path / "packed")
    folder = pipeline.prepare(job, echo=lambda *_: None)
    meta = json.loads((folder / "dataset.json").read_text())
    assert folder.name.startswith("text-") and meta["vocab_size"] == 257 and meta["stats"]["rows"] > 10
    assert pipeline.prepare(job, echo=lambda *_: None) == folder  # not prepared twice
    tr = Trainer(run, device="cpu", cache=tmp_path / "packed")
    feed = iter(tr.batches())
    first = next(feed)
    assert first.input_ids.shape == (4, 64) and first.loss_mask.any()
    assert (first.position_ids[:, 1:] <= first.position_ids[:, :-1]).any()  # several documents per row
    losses = [tr.train_step(b)["loss"].item() for b in [first] + [next(feed) for _ in range(7)]]
    assert losses[-1] < losses[0]
    again = next(iter(Trainer(run, device="cpu", cache=tmp_path / "packed").batches()))
    assert np.array_equal(again.input_ids, first.input_ids)  # batch i depends on the seed and i only


def test_chat_templates_render_prefixes_and_train_on_the_replies(tmp_path):
    """A Llama-3-style template (a beginning-of-text token once, headers per role) read from a
    tokenizer folder: what each message adds, and which characters a run trains on."""
    import json

    from bux_b200.data import templates

    source = ("{{ bos_token }}{% for m in messages %}<|start_header_id|>{{ m['role'] }}<|end_header_id|>\n\n"
              "{{ m['content'] | trim }}<|eot_id|>{% endfor %}"
              "{% if add_generation_prompt %}<|start_header_id|>assistant<|end_header_id|>\n\n{% endif %}")
    (tmp_path / "tokenizer_config.json").write_text(json.dumps(
        {"bos_token": {"content": "<|begin_of_text|>"}, "eos_token": "<|eot_id|>", "chat_template": source}))
    t = templates.load(str(tmp_path))
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": " hi "},
            {"role": "assistant", "content": "hello"}, {"role": "user", "content": "bye"},
            {"role": "assistant", "content": "ciao"}]
    whole = t.render(msgs)
    assert whole.startswith("<|begin_of_text|><|start_header_id|>system") and whole.count("<|begin_of_text|>") == 1
    assert t.render(msgs[:2], prompt=True).endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")
    pieces = t.pieces(msgs)
    assert "".join(p for p, _, _ in pieces) == whole
    assert [r for _, r, _ in pieces] == ["system", "user", "assistant", "user", "assistant"]
    text, role, start = pieces[2]
    assert text[start:] == "hello<|eot_id|>" and text[:start] == "<|start_header_id|>assistant<|end_header_id|>\n\n"
    assert pieces[1][2] == 0 and "hi<|eot_id|>" in pieces[1][0]          # trimmed as the template says
    # built-in and inline sources
    assert templates.load(None).render([{"role": "user", "content": "x"}], prompt=True).endswith("<|im_start|>assistant\n")
    assert templates.load("chatml").source == templates.CHATML
    assert templates.load("{{ messages | length }} turns").render(msgs) == "5 turns"
    import pytest

    with pytest.raises(ValueError):
        templates.load("no_such_template")


def test_chat_documents_mask_only_the_assistants_words(tmp_path):
    import json

    from bux_b200.config import training as T
    from bux_b200.data import documents as D
    from bux_b200.data.tokenizer import load as load_tokenizer

    rows = [{"messages": [{"role": "user", "content": "ab"}, {"role": "assistant", "content": "cd"},
                          {"role": "user", "content": "ef"}, {"role": "assistant", "content": "gh"}]}]
    path = tmp_path / "chat.jsonl"
    path.write_text("\n".join(json.dumps(r) for r in rows))
    tok = load_tokenizer(T.TokenizerConfig(name="bytes"))

    def trained(train_on):
        cfg = T.ChatConfig(path=str(path), train_on=train_on)
        (ids, mask), = list(D.chat(cfg, tok))
        return bytes(int(i) for i, m in zip(ids, mask) if m).decode()

    assert trained("assistant") == "cd<|im_end|>\ngh<|im_end|>\n"
    assert trained("last") == "gh<|im_end|>\n"
    assert trained("all").startswith("<|im_start|>user\nab")


class _Frame:
    """What `data.spark` uses of a Spark DataFrame, over one Arrow table held here."""

    def __init__(self, table, key=None):
        self.table, self.key = table, key

    def select(self, column):
        return _Frame(self.table.select([column]))

    def mapInArrow(self, fn, ddl):
        import pyarrow as pa

        from bux_b200.data import documents as D

        assert ddl == "key bigint, input_ids array<int>, loss_mask array<boolean>"
        # several small batches, as Spark hands a partition over
        batches = [b for piece in self.table.to_batches(max_chunksize=17) for b in fn([piece])]
        return _Frame(pa.Table.from_batches(batches, D.schema()))

    def persist(self):
        return self

    def agg(self, count, tokens):
        n = self.table.num_rows
        total = sum(len(x) for x in self.table.column("input_ids").to_pylist())
        return NS(first=lambda: (n, total or None))

    def groupBy(self, key):
        return _Frame(self.table, key)

    def applyInArrow(self, fn, ddl):
        import pyarrow as pa

        from bux_b200.data import packing as P

        assert ddl == "input_ids array<int>, position_ids array<int>, loss_mask array<boolean>"
        name, shift = self.key
        of = self.table.column(name).to_numpy() >> shift
        rng = np.random.default_rng(0)
        outs = []
        for c in sorted(set(of.tolist())):
            rows = np.nonzero(of == c)[0]
            rng.shuffle(rows)   # a shuffle delivers a group's rows in any order
            outs.append(fn((pa.scalar(c),), self.table.take(pa.array(rows))))
        return _Frame(pa.concat_tables(outs) if outs else P.schema().empty_table())

    @property
    def write(self):
        frame = self

        class W:
            def mode(self, m):
                assert m == "overwrite"
                return self

            def parquet(self, folder):
                import os

                import pyarrow.parquet as pq

                os.makedirs(folder, exist_ok=True)
                pq.write_table(frame.table, f"{folder}/part-00000-spark.parquet")

        return W()


_FUNCTIONS = NS(count=lambda c: ("count", c), size=lambda c: ("size", c), sum=lambda c: ("sum", c),
                shiftright=lambda c, n: NS(alias=lambda name: (c, n)))


def test_the_spark_engine_packs_the_rows_the_local_engine_packs(tmp_path):
    """`data.spark` against a stand-in for a Spark session (pyspark is not installed): the
    same `Job.map` and `Job.reduce` under mapInArrow / applyInArrow give the local engine's rows."""
    import pyarrow as pa
    import pyarrow.parquet as pq

    from bux_b200.config import training as T
    from bux_b200.data import pipeline, spark

    rng = np.random.default_rng(2)
    texts = [f"doc {i}: " + " ".join(rng.choice(["alpha", "beta", "gamma"], rng.integers(3, 40))) for i in range(300)]
    src = tmp_path / "docs.parquet"
    pq.write_table(pa.table({"text": texts}), src)
    job = pipeline.Job(T.TextConfig(path=str(src)), T.TokenizerConfig(name="bytes"),
                       T.BestFitPacking(chunk=4096), 64, str(tmp_path / "local"))
    local = pipeline.prepare(job, echo=lambda *_: None)
    meta = json.loads((local / "dataset.json").read_text())
    assert len(meta["parts"]) > 1   # several chunks: the grouping by key is exercised

    session = NS(read=NS(parquet=lambda path: _Frame(pq.read_table(path))))
    folder = spark.prepare(job, session, str(tmp_path / "spark"), functions=_FUNCTIONS)
    assert spark.prepare(job, session, str(tmp_path / "spark"), functions=_FUNCTIONS) == folder
    smeta = json.loads(open(f"{folder}/dataset.json").read())
    assert smeta["job"] == meta["job"] and smeta["vocab_size"] == meta["vocab_size"]
    assert smeta["stats"]["docs"] == 300 and smeta["parts"] == ["part-00000-spark.parquet"]

    def rows_of(folder, parts):
        t = pa.concat_tables([pq.read_table(f"{folder}/{p}") for p in parts])
        return sorted(zip(map(tuple, t.column("input_ids").to_pylist()), map(tuple, t.column("position_ids").to_pylist()),
                          map(tuple, t.column("loss_mask").to_pylist())))

    assert rows_of(local, meta["parts"]) == rows_of(folder, smeta["parts"])
    # the reader takes the Spark-written folder as it takes the local one
    train = NS(tokenizer=job.tokenizer, packing=job.packing, seq_len=64)
    a = prepared.Prepared(job.source, train, tmp_path / "spark", (0, 1), prepare_missing=False)
    assert a.total == meta["stats"]["rows"] and a.rows(0, 4).input_ids.shape == (4, 64)
