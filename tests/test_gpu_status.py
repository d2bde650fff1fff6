"""Failure detection on one GPU, the benign way: a bounded device wait that nothing
satisfies returns, records itself in the status word, and leaves the context usable.
Also: the trainer reads that word on the training path, and packed rows are masked by
document on the GPU."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_reports(cuda):
    from bux_b200.ops import kernels as K

    K.status_word(cuda).zero_()
    flags = torch.zeros(4, dtype=torch.int32, device=cuda)  # four "peers", none of which ever signals
    K.ep_wait(flags, epoch=1, limit_s=0.05)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match=r"kernel 4, site 2"):
        K.check_status(cuda, "test")
    K.check_status(cuda, "test")  # the word was cleared by the report
    # the context still works: the same wait succeeds once the flags are there
    flags.fill_(1)
    K.ep_wait(flags, epoch=1, limit_s=0.05)
    torch.cuda.synchronize()
    K.check_status(cuda, "test")


SRC = """
d_model=128
vocab_size=256
n = rmsnorm
a = gqa(num_heads=2, num_kv_heads=1, head_dim=64, rope=rope())
m = gated_mlp(intermediate_size=256, activation=swish)
model = embed ([n a] [n m])^2 n head
data = synthetic
optimizer = adamw(lr=1e-3)
seq_len = 256
batch = 2
steps = 4
precision = precision(compute=bfloat16)
"""


def test_trainer_reports_a_wait_that_ran_out(cuda):
    from bux_b200.lang import compile_runs
    from bux_b200.ops import kernels as K
    from bux_b200.train.trainer import KernelWaitError, Trainer

    run = compile_runs(SRC, filename="s.bux")[0]
    tr = Trainer(run, device=cuda)
    feed = iter(tr.batches())
    tr.train_step(next(feed))["loss"].item()
    tr.check_kernels("a clean step")  # nothing ran out
    flags = torch.zeros(2, dtype=torch.int32, device=cuda)
    K.ep_wait(flags, epoch=1, limit_s=0.02)  # a wait nobody satisfies, queued before the next step
    tr.train_step(next(feed))["loss"].item()
    with pytest.raises(KernelWaitError, match="kernel 4, site 2"):
        tr.check_kernels("step 2")
    assert tr.stopping
    tr.check_kernels("afterwards")  # reported once, then clean
    K.check_status(cuda, "test")


def test_packed_rows_are_masked_by_document_on_the_gpu(cuda):
    """A row packed with several documents trains like those documents apart: position
    ids that restart mark the boundaries, and the trainer must turn them into segment
    ids on the device (one step, loss compared with the documents as separate rows)."""
    from bux_b200.lang import compile_runs
    from bux_b200.train import data as D
    from bux_b200.train.trainer import Trainer, segments_of

    run = compile_runs(SRC, filename="s.bux", overrides=["batch = 1", "seq_len = 256"])[0]
    rng = np.random.default_rng(0)
    ids = rng.integers(0, 256, size=(1, 256), dtype=np.int32)
    lens = [64, 32, 96, 64]
    pos = np.concatenate([np.arange(n, dtype=np.int32) for n in lens])[None]
    packed = D.Batch(ids, pos, np.ones_like(ids, dtype=bool))
    seg = segments_of(torch.from_numpy(pos).long())
    assert seg[0, 0] == 1 and seg[0, 63] == 1 and seg[0, 64] == 2 and seg[0, -1] == 4

    def loss_of(batch, seed=3):
        tr = Trainer(run, device=cuda, seed=seed)
        return float(tr.train_step(batch)["loss"].item())

    got = loss_of(packed)
    # the same tokens, each document alone in a row (padded with masked positions)
    rows, start = [], 0
    total, count = 0.0, 0
    for n in lens:
        row = np.zeros((1, 256), dtype=np.int32)
        row[0, :n] = ids[0, start:start + n]
        mask = np.zeros((1, 256), dtype=bool)
        mask[0, :n] = True
        p = np.arange(256, dtype=np.int32)[None]
        one = loss_of(D.Batch(row, p, mask))
        total += one * (n - 1)
        count += n - 1
        start += n
    assert got == pytest.approx(total / count, rel=2e-2)
    # and it differs from reading the row as one document
    plain = loss_of(D.Batch(ids, np.arange(256, dtype=np.int32)[None], np.ones_like(ids, dtype=bool)))
    assert abs(plain - got) > 1e-4
