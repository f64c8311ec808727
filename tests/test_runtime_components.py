"""Host-side runtime pieces on CPU: schedules, micro-batch calculators, the re-run state machine with host-side
fault injection, data iterators, indexed / GPT / blended datasets against plain numpy oracles, the runtime
profiler's files, and configuration loading."""
import json
import math
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from hetu_galvatron_b200.runtime import rerun as rr  # noqa: E402
from hetu_galvatron_b200.runtime import scheduler as sch  # noqa: E402


class _Opt:
    def __init__(self):
        self.param_groups = [{"lr": 0.0, "weight_decay": 0.0}]
        self.lr, self.weight_decay = 0.0, 0.0


def _sched(style="cosine", **kw):
    args = dict(init_lr=0.0, max_lr=1e-3, min_lr=1e-4, lr_warmup_steps=100, lr_decay_steps=1000, lr_decay_style=style,
                start_wd=0.0, end_wd=0.1, wd_incr_steps=1000, wd_incr_style="linear")
    args.update(kw)
    return sch.OptimizerParamScheduler(_Opt(), **args)


def test_lr_schedules():
    s = _sched("cosine")
    s.step(50)
    assert s.get_lr() == pytest.approx(0.5e-3)
    s.step(50)
    assert s.get_lr() == pytest.approx(1e-3)
    s.step(450)  # half-way through the decay
    assert s.get_lr() == pytest.approx(1e-4 + 0.5 * 9e-4)
    s.step(10000)
    assert s.get_lr() == pytest.approx(1e-4)
    lin = _sched("linear")
    lin.step(550)
    assert lin.get_lr() == pytest.approx(1e-4 + 0.5 * 9e-4)
    const = _sched("constant")
    const.step(700)
    assert const.get_lr() == pytest.approx(1e-3)
    isq = _sched("inverse-square-root")
    isq.step(400)
    assert isq.get_lr() == pytest.approx(1e-3 * math.sqrt(100) / math.sqrt(400))
    wsd = _sched("WSD", wsd_decay_steps=200, lr_wsd_decay_style="linear")
    wsd.step(700)
    assert wsd.get_lr() == pytest.approx(1e-3)
    wsd.step(200)  # half of the tail
    assert wsd.get_lr() == pytest.approx(1e-4 + 0.5 * 9e-4)


def test_wd_schedule_and_state_roundtrip():
    s = _sched("cosine")
    s.step(250)
    assert s.get_wd() == pytest.approx(0.025)
    sd = json.loads(json.dumps(s.state_dict()))
    t = _sched("cosine")
    t.load_state_dict(sd)
    assert t.num_steps == 250 and t.get_lr() == pytest.approx(s.get_lr())
    assert s.optimizer.param_groups[0]["lr"] == pytest.approx(s.get_lr())


def test_scheduler_rejects_bad_arguments():
    with pytest.raises(AssertionError):
        _sched(lr_warmup_steps=2000)
    with pytest.raises(AssertionError):
        _sched(min_lr=1.0)
    with pytest.raises(AssertionError):
        _sched("WSD")


def test_microbatch_calculators():
    c = sch.build_num_microbatches_calculator(64, 2, 4)
    assert c.get() == 8 and c.get_current_global_batch_size() == 64
    r = sch.build_num_microbatches_calculator(64, 2, 4, [16, 16, 300])
    assert r.get_current_global_batch_size() == 16 and r.get() == 2
    r.update(150, True)
    assert r.get_current_global_batch_size() in (32, 48)
    r.update(1000, True)
    assert r.get_current_global_batch_size() == 64 and r.get() == 8
    with pytest.raises(AssertionError):
        sch.build_num_microbatches_calculator(60, 8, 4)


# ---- re-run state machine -------------------------------------------------------------------------------------
def _step(m, it, value_of):
    """One training step under the machine; returns how many times forward-backward ran."""
    runs = 0
    while m.should_run_forward_backward(it):
        batch = next(it)
        runs += 1
        m.validate_result(value_of(batch, runs), m.is_unexpectedly_large(10.0), "loss", tolerance=0.0)
    return runs


def test_rerun_disabled_and_clean_steps():
    m = rr.RerunStateMachine(rr.RerunMode.DISABLED)
    it = rr.RerunDataIterator(range(100))
    assert _step(m, it, lambda b, r: 1.0) == 1 and _step(m, it, lambda b, r: 1.0) == 1
    m = rr.RerunStateMachine(rr.RerunMode.VALIDATE_RESULTS)
    assert _step(m, it, lambda b, r: 1.0) == 1
    assert m.should_checkpoint_and_exit() == (False, False, 0)


def test_rerun_transient_fault_replays_the_same_batch():
    m = rr.RerunStateMachine(rr.RerunMode.VALIDATE_RESULTS)
    it = rr.RerunDataIterator(range(100))
    seen = []

    def value(b, run):
        seen.append(b)
        return float("nan") if run == 1 else 2.0

    assert _step(m, it, value) == 2
    assert seen == [0, 0]                                      # the re-run saw the same data
    assert m.log[-1][1] == rr.RerunDiagnostic.TRANSIENT_ERROR.value
    assert m.should_checkpoint_and_exit() == (False, False, 0)
    assert _step(m, it, lambda b, r: 1.0) == 1 and next(it) == 2


def test_rerun_reproducible_fault_asks_for_checkpoint_then_resolves(tmp_path):
    tracker = str(tmp_path / "rejected.json")
    m = rr.RerunStateMachine(rr.RerunMode.VALIDATE_RESULTS, result_rejected_tracker_filename=tracker)
    it = rr.RerunDataIterator(range(100))
    assert _step(m, it, lambda b, r: float("inf")) == 2      # same bad value twice
    save, leave, code = m.should_checkpoint_and_exit()
    assert (save, leave, code) == (True, True, rr.EXIT_CODE_RESUME_TO_DISAMBIGUATE)
    sd = json.loads(json.dumps(m.state_dict(it)))

    # "another device": restore, pretend the device id changed, the value differs -> persistent error on the first
    m2 = rr.RerunStateMachine(rr.RerunMode.VALIDATE_RESULTS, result_rejected_tracker_filename=tracker)
    it2 = rr.RerunDataIterator(range(100))
    m2.load_state_dict(sd, it2)
    m2._device = staticmethod(lambda: 7)
    assert _step(m2, it2, lambda b, r: 1.5) == 1
    assert m2.log[-1][1] == rr.RerunDiagnostic.PERSISTENT_ERROR.value
    assert m2.should_checkpoint_and_exit() == (False, True, rr.EXIT_CODE_FAILED_ON_RESULT_VALIDATION)

    # same value elsewhere -> the value is real; iteration recorded for skipping
    m3 = rr.RerunStateMachine(rr.RerunMode.VALIDATE_RESULTS, result_rejected_tracker_filename=tracker)
    it3 = rr.RerunDataIterator(range(100))
    m3.load_state_dict(sd, it3)
    m3._device = staticmethod(lambda: 7)
    assert _step(m3, it3, lambda b, r: float("inf")) == 1
    assert m3.log[-1][1] == rr.RerunDiagnostic.CORRECT_RESULT.value
    assert rr.get_skipped_iterations_from_tracker_file(tracker) == [0]


def test_rerun_injector_reaches_each_diagnosis():
    inj = rr.RerunErrorInjector(error_injection_rate=10 ** 6, error_injection_type=rr.RerunDiagnostic.TRANSIENT_ERROR)
    m = rr.RerunStateMachine(rr.RerunMode.VALIDATE_RESULTS, error_injector=inj)
    it = rr.RerunDataIterator(range(10))
    assert _step(m, it, lambda b, r: 1.0) == 2
    assert m.log[-1][1] == rr.RerunDiagnostic.TRANSIENT_ERROR.value
    inj = rr.RerunErrorInjector(error_injection_rate=10 ** 6, error_injection_type=rr.RerunDiagnostic.PERSISTENT_ERROR)
    m = rr.RerunStateMachine(rr.RerunMode.VALIDATE_RESULTS, error_injector=inj)
    assert _step(m, it, lambda b, r: 1.0) == 2
    assert m.should_checkpoint_and_exit()[2] == rr.EXIT_CODE_RESUME_TO_DISAMBIGUATE


def test_rerun_determinism_stats():
    m = rr.RerunStateMachine(rr.RerunMode.REPORT_DETERMINISM_STATS)
    it = rr.RerunDataIterator(range(10))
    assert _step(m, it, lambda b, r: 1.0 + 1e-3 * (r - 1)) == 2
    st = m.stats["loss"]
    assert "max" in st.print_stats()


# ---- datasets -------------------------------------------------------------------------------------------------
def _write_corpus(prefix, docs, dtype=np.uint16):
    from hetu_galvatron_b200.runtime.datasets.indexed import IndexedDatasetBuilder, bin_path, idx_path

    b = IndexedDatasetBuilder(bin_path(prefix), dtype=dtype)
    for d in docs:
        b.add_item(d)
        b.end_document()
    b.finalize(idx_path(prefix))


def _docs(n=60, seed=0, vocab=500):
    rng = np.random.RandomState(seed)
    return [rng.randint(1, vocab, size=rng.randint(5, 90)) for _ in range(n)]


def test_indexed_dataset_roundtrip(tmp_path):
    from hetu_galvatron_b200.runtime.datasets.indexed import IndexedDataset

    docs = _docs()
    prefix = str(tmp_path / "corpus")
    _write_corpus(prefix, docs)
    for mmap in (True, False):
        ds = IndexedDataset(prefix, mmap=mmap)
        assert len(ds) == len(docs) and ds.dtype == np.uint16
        assert list(ds.document_indices) == list(range(len(docs) + 1))
        for i in (0, 7, len(docs) - 1):
            assert np.array_equal(ds[i], docs[i])
        assert np.array_equal(ds.get(3, 2, 3), docs[3][2:5])


def test_sample_index_matches_python_oracle():
    from hetu_galvatron_b200.runtime.datasets.gpt import build_sample_idx, build_sample_idx_reference

    rng = np.random.RandomState(3)
    sizes = rng.randint(3, 70, size=200).astype(np.int32)
    for epochs, seq, drop in ((1, 32, True), (3, 17, True), (2, 64, False)):
        doc_idx = np.tile(np.arange(200, dtype=np.int32), epochs)
        rng.shuffle(doc_idx)
        tpe = int(sizes.sum())
        got = build_sample_idx(sizes, doc_idx, seq, epochs, tpe, drop, 1)
        want = build_sample_idx_reference(sizes, doc_idx, seq, epochs, tpe, drop, 1)
        assert got.shape == want.shape and np.array_equal(np.asarray(got, dtype=np.int64), want)


def test_gpt_dataset_samples_are_contiguous_token_windows(tmp_path):
    from hetu_galvatron_b200.runtime.datasets.gpt import GPTDataset, GPTDatasetConfig
    from hetu_galvatron_b200.runtime.datasets.indexed import IndexedDataset

    docs = _docs(80, seed=5)
    prefix = str(tmp_path / "c")
    _write_corpus(prefix, docs)
    cfg = GPTDatasetConfig(sequence_length=32, random_seed=11, path_to_cache=str(tmp_path / "cache"))
    ds = GPTDataset(IndexedDataset(prefix), prefix, np.arange(80, dtype=np.int32), 150, "train", cfg)
    assert len(ds) >= 150
    # the un-shuffled sample stream is the concatenation of the shuffled documents, windows overlap by one token
    stream = np.concatenate([docs[d] for d in ds.doc_index])
    inv = np.argsort(np.asarray(ds.shuffle_index))
    for k in (0, 1, 17, 149):
        s = ds[int(inv[k])]
        assert np.array_equal(s["tokens"].numpy(), stream[k * 32:(k + 1) * 32])
        assert np.array_equal(s["labels"].numpy(), stream[k * 32 + 1:(k + 1) * 32 + 1])
        assert s["loss_mask"].shape == (32,) and s["position_ids"][5] == 5
    # second construction hits the cache and gives the same samples
    ds2 = GPTDataset(IndexedDataset(prefix), prefix, np.arange(80, dtype=np.int32), 150, "train", cfg)
    assert torch.equal(ds2[3]["tokens"], ds[3]["tokens"])
    assert len(os.listdir(str(tmp_path / "cache"))) == 3


def _cold_cache_worker(payload):
    """One gloo rank: build the GPT dataset over a corpus whose index cache does not exist yet."""
    import torch.distributed as dist

    from hetu_galvatron_b200.runtime.datasets.gpt import GPTDataset, GPTDatasetConfig
    from hetu_galvatron_b200.runtime.datasets.indexed import IndexedDataset

    prefix, cache = payload["prefix"], payload["cache"]
    cfg = GPTDatasetConfig(sequence_length=32, random_seed=11, path_to_cache=cache)
    ds = GPTDataset(IndexedDataset(prefix), prefix, np.arange(80, dtype=np.int32), 400, "train", cfg)
    return {"rank": dist.get_rank(), "len": len(ds), "sample": ds[7]["tokens"].tolist(),
            "files": sorted(os.listdir(cache))}


def test_dataset_index_cache_is_built_once_by_rank_zero(tmp_path):
    """Four ranks start with a cold cache: rank 0 builds and publishes the index files atomically, the others wait at
    the barrier and map the finished files; everybody sees the same samples and no temporary file is left."""
    from tests.dist_utils import run_distributed

    prefix = str(tmp_path / "c")
    _write_corpus(prefix, _docs(80, seed=5))
    cache = str(tmp_path / "cache")
    res = run_distributed(__file__, "cold_cache", 4, {"prefix": prefix, "cache": cache}, timeout=120)
    assert len({r["len"] for r in res}) == 1 and all(r["sample"] == res[0]["sample"] for r in res)
    assert all(len(r["files"]) == 3 and not any(".tmp." in f for f in r["files"]) for r in res)


def _fd_exchange_worker(payload):
    """One gloo rank: pass an open file to every other rank over the allocator's descriptor exchange."""
    import torch.distributed as dist

    from hetu_galvatron_b200.parallel.symm_vmm import _exchange_fds

    me = dist.get_rank()
    path = os.path.join(payload["dir"], "rank%d.txt" % me)
    with open(path, "w") as f:
        f.write("written by rank %d" % me)
    fd = os.open(path, os.O_RDONLY)
    seen = {}
    for tag in ("first", "second"):          # two rounds: the socket names of a round are gone before the next
        got = _exchange_fds(fd, dist.group.WORLD, tag)
        assert got[me] == -1
        for r, other in enumerate(got):
            if r != me:
                # the received descriptor shares its file offset with every other copy: read at an explicit position
                seen["%s_%d" % (tag, r)] = os.pread(other, 64, 0).decode()
                os.close(other)
    os.close(fd)
    return seen


def test_vmm_allocator_passes_descriptors_between_ranks(tmp_path):
    """The descriptor exchange behind ``HG_SYMM_ALLOC=vmm`` (abstract Unix sockets, SCM_RIGHTS): every rank ends up with
    a working descriptor of every other rank's file, in rank order."""
    from tests.dist_utils import run_distributed

    res = run_distributed(__file__, "fd_exchange", 3, {"dir": str(tmp_path)}, timeout=120)
    for me, seen in enumerate(res):
        for tag in ("first", "second"):
            for r in range(3):
                if r != me:
                    assert seen["%s_%d" % (tag, r)] == "written by rank %d" % r


def test_nonzero_device_status_rejects_the_step(monkeypatch):
    """A kernel whose bounded wait ran out leaves a code in the device status word; the training loop reads it once
    per iteration and raises instead of keeping the step."""
    from hetu_galvatron_b200.ops._lib import KernelError
    from hetu_galvatron_b200.runtime import trainer

    trainer.check_device_status(torch.device("cpu"))          # healthy: no error
    monkeypatch.setattr(trainer, "_device_status_code", lambda device: 5)
    with pytest.raises(KernelError, match="peer flag"):
        trainer.check_device_status(torch.device("cpu"))
    # and the loop calls it: a one-layer model, first iteration
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs

    args = GalvatronRuntimeArgs(
        parallel=dict(mixed_precision="fp32"),
        model=dict(model_size="llama-test", hidden_size=64, num_layers=1, num_attention_heads=2, ffn_hidden_size=128,
                   vocab_size=128, make_vocab_size_divisible_by=8, normalization="RMSNorm",
                   activation_func="torch.nn.functional.silu", gated_linear_unit=True),
        train=dict(seq_length=16, global_batch_size=2, chunks=1, lr=1e-3, train_iters=2),
        data=dict(use_random_dataset=True))
    with pytest.raises(KernelError):
        trainer.train(args, max_iters=2)


def test_training_loop_evaluates_on_the_validation_split(tmp_path, capsys):
    """With a corpus on disk the loop sets do_train / do_valid, runs ``eval_iters`` forward-only batches of the
    validation split every ``eval_interval`` iterations and reports their mean loss; evaluation leaves no gradients."""
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
    from hetu_galvatron_b200.runtime import trainer

    prefix = str(tmp_path / "c")
    _write_corpus(prefix, _docs(400, seed=9))
    args = GalvatronRuntimeArgs(
        parallel=dict(mixed_precision="fp32"),
        model=dict(model_size="llama-test", hidden_size=64, num_layers=1, num_attention_heads=2, ffn_hidden_size=128,
                   vocab_size=128, make_vocab_size_divisible_by=8, normalization="RMSNorm",
                   activation_func="torch.nn.functional.silu", gated_linear_unit=True),
        train=dict(seq_length=16, global_batch_size=2, chunks=1, lr=1e-3, train_iters=4, eval_interval=2, eval_iters=2),
        data=dict(data_path=[prefix], split="8,1,1", path_to_cache=str(tmp_path / "cache")))
    losses = trainer.train(args, max_iters=4)
    out = capsys.readouterr().out
    assert len(losses) == 4 and args.train.do_train and args.train.do_valid
    assert out.count("validation loss") == 2


def _pp_eval_worker(payload):
    """One gloo rank of a two-stage pipeline: a few training iterations with periodic evaluation."""
    import contextlib
    import io

    import torch.distributed as dist

    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
    from hetu_galvatron_b200.runtime import trainer

    args = GalvatronRuntimeArgs(
        parallel=dict(mixed_precision="fp32", pp_deg=2, pipeline_type="pipedream_flush"),
        model=dict(model_size="llama-test", hidden_size=64, num_layers=2, num_attention_heads=2, ffn_hidden_size=128,
                   vocab_size=128, make_vocab_size_divisible_by=8, normalization="RMSNorm",
                   activation_func="torch.nn.functional.silu", gated_linear_unit=True),
        train=dict(seq_length=16, global_batch_size=4, chunks=2, lr=1e-3, train_iters=4, eval_interval=2, eval_iters=1),
        data=dict(data_path=[payload["prefix"]], split="8,1,1", path_to_cache=payload["cache"]),
        rank=dist.get_rank(), world_size=2)
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        losses = trainer.train(args, max_iters=4)
    return {"losses": losses, "validation_lines": buf.getvalue().count("validation loss")}


def test_evaluation_under_pipeline_parallelism(tmp_path):
    """Forward-only evaluation through a two-stage pipeline: the last stage holds and reports the validation loss."""
    from tests.dist_utils import run_distributed

    prefix = str(tmp_path / "c")
    _write_corpus(prefix, _docs(400, seed=9))
    res = run_distributed(__file__, "pp_eval", 2, {"prefix": prefix, "cache": str(tmp_path / "cache")}, timeout=180)
    assert res[0]["validation_lines"] == 0 and res[1]["validation_lines"] == 2
    assert all(l is None for l in res[0]["losses"]) and all(l is not None for l in res[1]["losses"])


def test_blended_dataset_follows_weights():
    from hetu_galvatron_b200.runtime.datasets.blended import BlendedDataset

    class D(torch.utils.data.Dataset):
        def __init__(self, tag, n):
            self.tag, self.n = tag, n

        def __len__(self):
            return self.n

        def __getitem__(self, i):
            return {"tokens": torch.tensor([self.tag, i])}

    b = BlendedDataset([D(0, 1000), D(1, 1000), D(2, 1000)], [0.5, 0.3, 0.2], 1000)
    counts = np.bincount(b.dataset_index, minlength=3)
    assert list(counts) == [500, 300, 200]
    for prefix in (10, 100, 333):  # greedy: every prefix tracks the weights within one sample
        c = np.bincount(b.dataset_index[:prefix], minlength=3)
        assert np.all(np.abs(c - np.array([0.5, 0.3, 0.2]) * prefix) <= 1.0 + 1e-9)
    item = b[10]
    assert item["dataset_id"] == int(b.dataset_index[10]) and item["tokens"][1] == int(b.dataset_sample_index[10])
    ex = BlendedDataset([D(0, 5), D(1, 10)], None, None)
    assert len(ex) == 15 and list(np.bincount(ex.dataset_index)) == [5, 10]


def test_builder_splits_and_collate(tmp_path):
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
    from hetu_galvatron_b200.runtime.datasets import builder

    assert builder.parse_weighted_paths(["0.3", "a", "0.7", "b"]) == (["a", "b"], [0.3, 0.7])
    assert builder.parse_weighted_paths(["a"]) == (["a"], None)
    sp = builder.parse_split("90,10,0")
    assert sp[0] == (0.0, 0.9) and sp[1] == pytest.approx((0.9, 1.0)) and sp[2] is None
    prefix = str(tmp_path / "c")
    _write_corpus(prefix, _docs(100, seed=9))
    args = GalvatronRuntimeArgs(model=dict(model_size="llama-test", hidden_size=64, num_layers=1, num_attention_heads=2, vocab_size=512),
                                train=dict(seq_length=16, global_batch_size=4, train_iters=10, eval_iters=2, eval_interval=5),
                                data=dict(data_path=[prefix], split="90,10,0", data_cache_path=str(tmp_path / "cache")))
    tr, va, te = builder.build_train_valid_test_datasets(args)
    assert len(tr) >= 40 and va is not None and te is None
    tokens, kw, _ = builder.gpt_collate_fn([tr[0], tr[1]])
    assert tokens.shape == (2, 16) and kw["labels"].shape == (2, 16) and kw["loss_mask"].shape == (2, 16)


def test_samplers_partition_the_batch():
    from hetu_galvatron_b200.runtime.data import PretrainingRandomSampler, PretrainingSampler

    per_rank = [list(PretrainingSampler(64, 8, 2, r, 4)) for r in range(4)]
    first = sorted(sum((pr[0] for pr in per_rank), []))
    assert first == list(range(8, 16)) and len(per_rank[0]) == 7
    rnd = [list(PretrainingRandomSampler(64, 64, 0, 2, r, 4, data_sharding=True, seed=1)) for r in range(4)]
    seen = sorted(sum((sum(pr, []) for pr in rnd), []))
    assert seen == list(range(64))


# ---- runtime profiler ----------------------------------------------------------------------------------------
def test_runtime_profiler_files(tmp_path):
    from hetu_galvatron_b200.profiler import runtime as prof

    assert prof.memory_strategy_key(1, 2, 8, False, True, 2).startswith("1_2_4")
    p = str(tmp_path / "mem.json")
    prof.save_profiled_memory(p, 1, 2, 8, [1], 8, 0, 100.0, 50.0, 75.0, 0, True, 2, 4096)
    prof.save_profiled_memory(p, 1, 2, 8, [1], 8, 7, 90.0, 40.0, 70.0, 0, True, 2, 4096)
    cfg = json.load(open(p))
    (key, val), = cfg.items()
    assert "layernum1_bsz8_seq4096_rank0_ms" in val and "layernum1_bsz8_seq4096_rank7_act_peak" in val
    t = str(tmp_path / "time.json")
    prof.save_profiled_time(t, 12.5, 8, [2], 4096)
    assert json.load(open(t)) == {"layernum2_bsz8_seq4096": 12.5}


def test_runtime_profiler_time_filter():
    from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
    from hetu_galvatron_b200.profiler.runtime import RuntimeProfiler

    args = GalvatronRuntimeArgs(model=dict(model_size="llama-test", hidden_size=64, num_layers=1, num_attention_heads=2, vocab_size=512),
                                train=dict(seq_length=16, global_batch_size=4))
    p = RuntimeProfiler(args)
    p.set_time_profiler(0, 100)
    p.time_list = [10.0] * 20 + [200.0]
    f = p.filtered_time_samples()
    assert 200.0 not in f and p.average_time() == pytest.approx(10.0)


# ---- configuration ----------------------------------------------------------------------------------------------
def test_config_loader_overrides_and_zoo(tmp_path):
    from hetu_galvatron_b200.config import loader
    from hetu_galvatron_b200.config.model_config import model_name, resolve_model_config

    y = tmp_path / "train.yaml"
    y.write_text("runtime:\n  model:\n    model_size: llama2-7b\n  train:\n    seq_length: 2048\n    global_batch_size: 16\n"
                 "  parallel:\n    pp_deg: 2\n    global_tp_deg: ${runtime.parallel.pp_deg}\n")
    args = loader.load_config(str(y), ["runtime.train.seq_length=4096", "runtime.parallel.sdp=1"], mode="train_dist")
    assert args.train.seq_length == 4096 and args.parallel.pp_deg == 2 and args.parallel.global_tp_deg == 2
    assert args.parallel.sdp == 1
    resolve_model_config(args)
    assert args.model.hidden_size == 4096 and args.model.num_layers == 32
    assert "llama" in model_name(args)
    ov = loader.legacy_cli_to_overrides(["--pp_deg", "4", "--global_train_batch_size", "32", "--use-flash-attn"])
    assert "++runtime.parallel.pp_deg=4" in ov and "++runtime.train.global_batch_size=32" in ov


# ---- random streams ---------------------------------------------------------------------------------------------
def test_rng_tracker_streams():
    from hetu_galvatron_b200.parallel import random as rnd

    class G:
        def __init__(self, size, rank):
            self.size, self.rank = size, rank

    t = rnd.set_seed_with_group([G(2, 1), G(2, 1), G(4, 3)], [G(8, 5)], seed=1234, cuda=False)
    assert sorted(t.states_) == ["data-parallel-rng", "expert-parallel-rng-8", "model-parallel-rng-2", "model-parallel-rng-4"]
    before = torch.get_rng_state()
    with t.fork("model-parallel-rng-2"):
        a = torch.rand(4)
    assert torch.equal(torch.get_rng_state(), before)            # the default stream is untouched by the region
    with t.fork("model-parallel-rng-2"):
        b = torch.rand(4)
    assert not torch.equal(a, b)                                 # the named stream advances
    t2 = rnd.set_seed_with_group([G(2, 1)], None, 1234, cuda=False)
    with t2.fork("model-parallel-rng-2"):
        c = torch.rand(4)
    assert torch.equal(a, c)                                     # same seed, same rank -> same stream
    t3 = rnd.set_seed_with_group([G(2, 0)], None, 1234, cuda=False)
    with t3.fork("model-parallel-rng-2"):
        d = torch.rand(4)
    assert not torch.equal(a, d)                                 # another rank of the group differs
    with pytest.raises(ValueError):
        t3.add("again", 1234)
    with pytest.raises(KeyError):
        with t3.fork("missing"):
            pass


# ---- resharding index algebra ------------------------------------------------------------------------------------
@pytest.mark.parametrize("src,dst", [((1, 1), (2, 1)), ((4, 1), (2, 1)), ((1, 2), (2, 1)), ((2, 2), (1, 1)),
                                     ((2, 1), (1, 4)), ((1, 4), (4, 1)), ((2, 2), (4, 1))])
def test_reshard_pull_lists_match_the_collective_formulation(src, dst):
    """For every rank of a block, the (rank, row) list of the one-kernel resharding selects exactly the rows that
    "gather sequence -> undo zig-zag -> re-split batch -> zig-zag -> slice" produces."""
    from hetu_galvatron_b200.parallel.reshard import apply_zigzag, pull_lists

    def held(full, width, cp, i):
        return apply_zigzag(full, cp).chunk(width * cp, dim=0)[i].contiguous()

    S, H = 32, 1
    g_s, g_d = src[0] * src[1], dst[0] * dst[1]
    big = max(g_s, g_d)
    samples = 4 * big
    data = torch.arange(S * samples, dtype=torch.float32).view(S, samples, H)
    b_s, b_d = samples // (big // g_s), samples // (big // g_d)
    srcs = [held(data[:, (j // g_s) * b_s:(j // g_s + 1) * b_s], src[0], src[1], j % g_s).reshape(-1, H) for j in range(big)]
    flat = torch.stack(srcs)
    for j in range(big):
        want = held(data[:, (j // g_d) * b_d:(j // g_d + 1) * b_d], dst[0], dst[1], j % g_d)
        peer, row = pull_lists(S, S // g_d, b_d, b_s, j, src, dst, "cpu")
        assert torch.equal(flat[peer.long(), row.long()].view(S // g_d, b_d, H), want)


# ---- MoE router extras ---------------------------------------------------------------------------------------------
def test_sinkhorn_balances_and_routes():
    from hetu_galvatron_b200.models import moe

    torch.manual_seed(0)
    logits = torch.randn(64, 8) + torch.tensor([3.0, 0, 0, 0, 0, 0, 0, 0])   # expert 0 is everybody's favourite
    norm = moe.sinkhorn(logits)
    assert torch.allclose(norm.sum(0), torch.full((8,), 1 / 8), atol=2e-3)      # balanced columns
    probs, idx = moe.sinkhorn_routing(logits.clone().requires_grad_(), 2, training=True)
    greedy = logits.topk(2, dim=1).indices
    assert (idx == 0).sum() < (greedy == 0).sum()                               # fewer tokens pile on expert 0
    assert probs.requires_grad and torch.allclose(probs, torch.softmax(logits, -1).gather(1, idx))
    p1, i1 = moe.sinkhorn_routing(logits, 1, training=False)
    assert torch.equal(i1, torch.sigmoid(logits).topk(1, dim=1).indices)


def test_sequence_aux_loss_matches_per_sequence_formula():
    from hetu_galvatron_b200.models import moe

    torch.manual_seed(1)
    S, B, E, k = 16, 3, 4, 2
    logits = torch.randn(S * B, E)
    idx = logits.topk(k, dim=1).indices
    got = moe.sequence_aux_loss(logits, idx, E, k, 0.01, B)
    sc = torch.softmax(logits, -1).view(S, B, E)
    want = 0.0
    for b in range(B):
        counts = torch.bincount(idx.view(S, B, k)[:, b].reshape(-1), minlength=E).float()
        want += (sc[:, b].mean(0) * counts / (S * k)).sum() * E * 0.01
    assert got.item() == pytest.approx(float(want) / B, rel=1e-5)


def test_expert_bias_update_moves_towards_balance():
    from types import SimpleNamespace

    from hetu_galvatron_b200.models import moe

    r = moe.GalvatronMoERouter.__new__(moe.GalvatronMoERouter)
    torch.nn.Module.__init__(r)
    r.router = torch.nn.Module()
    r.router.register_buffer("expert_bias", torch.zeros(4))
    r.router.register_buffer("local_tokens_per_expert", torch.tensor([10.0, 2.0, 4.0, 4.0]))
    r.update_expert_bias(0.1)
    assert torch.allclose(r.router.expert_bias, torch.tensor([-0.1, 0.1, 0.1, 0.1]))
    assert float(r.router.local_tokens_per_expert.sum()) == 0.0


if __name__ == "__main__":
    from tests.dist_utils import worker_main

    worker_main({"cold_cache": _cold_cache_worker, "fd_exchange": _fd_exchange_worker, "pp_eval": _pp_eval_worker})
