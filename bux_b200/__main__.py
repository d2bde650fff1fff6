"""``bux COMMAND FILE [SETTING=VALUE ...]``: the command line.

Commands (reference: ``__main__.py:322-656``, table in ``docs/reference/cli.md:9-21``):
check, plan, fmt, json, render, train, launch, results, prepare, export, studio.
Trailing statements are appended to the file as overrides (``steps=100``,
``'optimizer = muon(lr=0.02)'``). ``check``, ``plan``, ``fmt``, ``json`` and
``render`` import no ML library.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def _parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="bux", description="LM ablations on B200s")
    sub = p.add_subparsers(dest="command", required=True)
    for name, doc in (("check", "type-check a file"), ("plan", "list a file's runs and their sizes"),
                      ("fmt", "print every run's canonical source"), ("json", "print every run's IR"),
                      ("render", "draw the model"), ("train", "train every run, one after another"),
                      ("launch", "train every run, sweeps over the GPUs"),
                      ("results", "tabulate the runs' metrics"), ("prepare", "tokenize and pack the data")):
        s = sub.add_parser(name, help=doc)
        s.add_argument("file")
        s.add_argument("overrides", nargs="*", help="statements that redefine the file's own")
        s.add_argument("--entry", default="model")
        s.add_argument("--only", default=None, help="keep the runs whose name contains TEXT")
        s.add_argument("--index", type=int, default=None, help="keep the run at this index of `plan`")
        if name == "render":
            s.add_argument("--expand", action="store_true", help="draw every block in place, not under its own name")
            s.add_argument("--outline", action="store_true", help="one layer per line, with the widths")
        if name in ("train", "launch", "results", "prepare"):
            s.add_argument("--out", default="runs")
            s.add_argument("--cache", default=".")
        if name in ("train", "launch"):
            s.add_argument("--device", default=None)
            s.add_argument("--quiet", action="store_true")
    e = sub.add_parser("export", help="export a trained run (or a file's model without weights) for transformers / vLLM")
    e.add_argument("run_dir", help="a run's directory, or a .bux file")
    e.add_argument("out")
    e.add_argument("overrides", nargs="*", help="with a file: statements that redefine the file's own")
    e.add_argument("--entry", default="model")
    e.add_argument("--step", type=int, default=None)
    e.add_argument("--dtype", default="bfloat16")
    e.add_argument("--check", action="store_true")
    st = sub.add_parser("studio", help="edit and watch a file in the browser")
    st.add_argument("file")
    st.add_argument("--port", type=int, default=8765, help="the first port tried (the next few when it is taken)")
    st.add_argument("--host", default="127.0.0.1")
    st.add_argument("--out", default="runs", help="where trainings started from the page put their runs")
    st.add_argument("--no-browser", action="store_true", help="print the URL only")
    return p


def _runs(args):
    from .lang import compile_runs

    source = Path(args.file).read_text()
    runs = compile_runs(source, entry=args.entry, filename=args.file, overrides=args.overrides)
    if args.only:
        runs = [r for r in runs if args.only in r.name]
    if args.index is not None:
        runs = [runs[args.index]]
    return runs


def _si(n: float) -> str:
    from .train.curriculum import si

    return si(n)


def _bytes(n: float) -> str:
    for unit, scale in (("GiB", 2 ** 30), ("MiB", 2 ** 20), ("KiB", 2 ** 10)):
        if n >= scale:
            return f"{n / scale:.3g}{unit}"
    return f"{n:.0f}B"


def plan_rows(runs) -> list:
    """One row per run: id, params, tokens, FLOPs/token, GPUs, memory per GPU, bubble.
    Nothing here touches a device (parameters are counted on the meta device)."""
    from .parallel import mesh as M
    from .train import curriculum
    from .train.flops import flops_per_token
    from .train.trainer import count_params

    rows = []
    for run in runs:
        t = run.train
        params = count_params(run.arch)
        tokens = curriculum.tokens(curriculum.stretches(t), t.steps)
        gpus = M.size(t.mesh)
        shards = M.param_shards(t.mesh, t.layout)
        stage = t.mesh.stage
        per_gpu = params * 4 / max(1, shards)
        moments = 4 if t.precision.moments == "float32" else 2
        optim_gpu = params * 2 * moments / max(1, shards)
        micro = max(t.methods.microbatches, 1)
        bubble = (stage - 1) / (micro * t.methods.rounds + stage - 1) if stage > 1 else 0.0
        rows.append((run.id, _si(params), _si(tokens), f"{tokens / params:.1f}",
                     _si(flops_per_token(run.arch, t.seq_len)), str(gpus), _bytes(per_gpu),
                     _bytes(optim_gpu), f"{bubble:.0%}", run.name))
    return rows


def _table(header, rows) -> str:
    widths = [max(len(str(x)) for x in col) for col in zip(header, *rows)]
    lines = ["  ".join(str(h).ljust(w) for h, w in zip(header, widths)).rstrip()]
    for r in rows:
        lines.append("  ".join(str(x).ljust(w) for x, w in zip(r, widths)).rstrip())
    return "\n".join(lines)


def main(argv=None) -> int:
    from .lang import BuxError

    args = _parser().parse_args(argv)
    try:
        return _dispatch(args)
    except BuxError as err:
        print(err, file=sys.stderr)
        return 1


def check_summary(report) -> list:
    """What ``bux check`` prints for a file without mistakes: the width, the vocabulary and the
    layers by type; for a run its budget, optimizer, schedule and data; for a sweep its axes
    (``docs/language/tooling.md`` there: `bux check`). A file without a model is a module and
    lists what it defines."""
    from collections import Counter

    from .lang import ir
    from .lang.printer import config_to_source

    if report.defines is not None:
        return ["a module: it defines " + ", ".join(report.defines) + ", and no model"]
    lines = []
    arch, train = report.arch, report.train
    if arch is not None:
        kinds = Counter((l.config.fn if l.config.type == "act" else l.config.type) for l in ir.unrolled_layers(arch.graph))
        lines.append(f"d_model={arch.d_model} vocab_size={arch.vocab_size} layers={sum(kinds.values())}")
        lines.append("  ".join(f"{kind}×{n}" for kind, n in kinds.most_common()))
    if train is not None:
        tokens = train.steps * train.batch * train.seq_len
        lines.append(f"{train.steps} steps × {train.batch} × {train.seq_len} tokens = {_si(tokens)} tokens")
        lines.append(f"optimizer={config_to_source(train.optimizer)} schedule={config_to_source(train.schedule)}")
        lines.append(f"data={config_to_source(train.data)}")
    if report.axes:
        axes = " × ".join(f"{a.where} ({' | '.join(str(o) for o in a.options)})" for a in report.axes)
        lines.append(f"sweep: {report.runs} runs over {axes}")
    for d in report.dimensions:
        lines.append(f"search: {d.where} = {config_to_source(d.space)}")
    return lines


def _dispatch(args) -> int:
    cmd = args.command
    if cmd == "check":
        from .lang import check

        report = check(Path(args.file).read_text(), entry=args.entry, filename=args.file,
                       overrides=args.overrides)
        for err in report.errors:
            print(err, file=sys.stderr)
            print(file=sys.stderr)
        if report.errors:
            print(f"{len(report.errors)} error(s)", file=sys.stderr)
            return 1
        for line in check_summary(report):
            print(line)
        return 0
    if cmd == "plan":
        runs = _runs(args)
        print(f"{len(runs)} run{'s' if len(runs) != 1 else ''}")
        print(_table(("id", "params", "tokens", "tok/param", "flops/tok", "gpus", "params/gpu",
                      "optim/gpu", "bubble", "run"), plan_rows(runs)))
        return 0
    if cmd in ("fmt", "json"):
        from .lang import BuxError, compile
        from .lang.printer import run_to_source, to_source

        try:
            runs = _runs(args)
        except BuxError as err:
            if "defines a model, not a run" not in err.message:
                raise
            # a model file: its architecture alone
            path = Path(args.file)
            arch = compile(path.read_text(), filename=str(path), entry=args.entry, overrides=args.overrides)
            print(to_source(arch) if cmd == "fmt" else arch.model_dump_json(indent=2), end="" if cmd == "fmt" else "\n")
            return 0
        if cmd == "fmt":
            print("\n".join(run_to_source(r) for r in runs), end="")
        else:
            import json as _json

            print(_json.dumps([r.model_dump(mode="json") for r in runs], indent=2))
        return 0
    if cmd == "render":
        from .lang import BuxError, compile
        from .lang.render import outline, render

        try:
            archs = [r.arch for r in _runs(args)[:1]]
        except BuxError as err:
            if "defines a model, not a run" not in err.message:
                raise
            # a model file draws as well as a run's
            path = Path(args.file)
            archs = [compile(path.read_text(), filename=str(path), entry=args.entry, overrides=args.overrides)]
        for arch in archs:
            print(outline(arch) if args.outline else render(arch, expand=args.expand), end="" if not args.outline else "\n")
        return 0
    if cmd == "train":
        # one process, or one rank of a job started by torchrun / srun / mpirun: `train_here`
        # joins the job the environment describes and shards the run over its mesh
        from .launch import train_here

        for run in _runs(args):
            train_here(run, out=args.out, cache=args.cache, device=args.device, quiet=args.quiet)
        return 0
    if cmd == "launch":
        from .launch import launch

        return launch(args.file, overrides=args.overrides, out=args.out, cache=args.cache,
                      only=args.only, index=args.index, entry=args.entry, device=args.device)
    if cmd == "results":
        from .launch import results

        print(results(_runs(args), args.out))
        return 0
    if cmd == "prepare":
        from .data import pipeline

        for run in _runs(args):
            for job in pipeline.jobs(run.train, args.cache):
                pipeline.prepare(job)
        return 0
    if cmd == "export":
        from .export import export

        if str(args.run_dir).endswith(".bux") and Path(args.run_dir).is_file():
            from .export import export_architecture

            export_architecture(args.run_dir, args.out, args.overrides, args.entry, args.dtype)
            return 0
        export(args.run_dir, args.out, step=args.step, dtype=args.dtype, check=args.check)
        return 0
    if cmd == "studio":
        from .studio import serve

        serve(args.file, port=args.port, out=args.out, host=args.host, browser=not args.no_browser)
        return 0
    raise AssertionError(cmd)


if __name__ == "__main__":
    sys.exit(main())
