"""The prepare pipeline on Spark: the map runs as ``mapInArrow``, the reduce as a grouped
``applyInArrow``.

    from pyspark.sql import SparkSession
    from bux_b200.data import spark
    from bux_b200.data.pipeline import jobs
    from bux_b200.lang import compile_runs

    [run] = compile_runs(open("examples/experiments/speedrun.bux").read())
    session = SparkSession.builder.getOrCreate()
    for job in jobs(run.train):
        spark.prepare(job, session, "s3://bucket/packed")

Both functions are the ones the local engine calls (`Job.map`, `Job.reduce`), and the
chunk of a document is the same function of its key, so a chunk holds the same rows
under either engine; which parquet file holds a chunk is Spark's choice. pyspark is
imported only by the calls that need it: the module imports without it.
Reference: ``data/spark.py:31-97``.
"""

from __future__ import annotations

import json

from . import documents as D
from . import packing as P
from . import tokenizer as TK
from .pipeline import Job, shift


def ddl(schema) -> str:
    """`schema` (Arrow) as a Spark DDL string: the result type of an Arrow function."""
    import pyarrow as pa

    names = {pa.int64(): "bigint", pa.int32(): "int", pa.bool_(): "boolean", pa.string(): "string"}

    def one(t):
        return f"array<{one(t.value_type)}>" if pa.types.is_list(t) else names[t]

    return ", ".join(f"{f.name} {one(f.type)}" for f in schema)


def rows(job: Job, records, functions=None):
    """The packed rows of `records` (a DataFrame that has the source's column) as a
    DataFrame in `packing.schema()`, with the counts of documents and tokens. The documents
    are counted before they are grouped (the count fixes the number of chunks), so they are
    persisted between the map and the reduce."""
    import pyarrow as pa

    F = functions
    if F is None:
        from pyspark.sql import functions as F
    docs = records.select(job.source.column).mapInArrow(job.map, ddl(D.schema())).persist()
    counted = docs.agg(F.count("*"), F.sum(F.size("input_ids"))).first()
    n, tokens = (int(counted[0]), int(counted[1] or 0)) if counted else (0, 0)
    chunks = job.chunks(tokens)

    def reduce(key, table):
        k = key[0]
        batches, _ = job.reduce(int(k.as_py() if hasattr(k, "as_py") else k), table)
        return pa.Table.from_batches(batches, P.schema())

    chunk = F.shiftright("key", shift(chunks)).alias("chunk")
    return docs.groupBy(chunk).applyInArrow(reduce, ddl(P.schema())), {"docs": n, "tokens": tokens}


def prepare(job: Job, session, cache: str, functions=None) -> str:
    """Write `job`'s dataset under `cache` (any URI Spark and Arrow can both write, such as
    ``s3://bucket/packed``) in the local engine's layout: parquet parts of rows and a
    ``dataset.json`` written last. A dataset that is whole already is returned at once;
    parts left by a write that failed are written over. Returns the dataset's folder."""
    import pyarrow.fs as pafs

    folder = f"{cache.rstrip('/')}/{job.name}"
    fs, path = pafs.FileSystem.from_uri(folder) if "://" in folder else (pafs.LocalFileSystem(), folder)
    if fs.get_file_info(f"{path}/dataset.json").type != pafs.FileType.NotFound:
        return folder
    out, stats = rows(job, session.read.parquet(job.source.path), functions)
    out.write.mode("overwrite").parquet(folder)
    listed = fs.get_file_info(pafs.FileSelector(path))
    parts = sorted(i.base_name for i in listed if i.base_name.endswith(".parquet"))
    meta = {"job": job.spec(), "files": [job.source.path], "parts": parts,
            "vocab_size": TK.load(job.tokenizer).vocab_size, "stats": stats}
    with fs.open_output_stream(f"{path}/dataset.json") as f:
        f.write(json.dumps(meta, indent=1).encode())
    return folder
