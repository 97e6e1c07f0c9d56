"""Training entry point: `python -m torch.distributed.run ... -m superscaler_b200.runtime.pretrain
--flexpipe-config plan.json --train-iters 3 --log-path logs/` (one rank per GPU).

Counterpart of the reference's pretrain_gpt.py / pretrain_t5.py / pretrain_resnet.py + training loop
(runtime/pretrain_gpt.py, runtime/megatron/training.py:83-168,925-1018): the model family comes from the plan
JSON, batches are synthetic, and at the last iteration every rank writes
`{log-path}/csv/{config}_stage{s}_rank{r}.csv` with the per-region times (ms) and memory (MB) that the
result-collection tools read (training.py:903-908).
"""
from __future__ import annotations

import argparse
import csv
import contextlib
import json
import math
import os
import sys
import time

import torch
import torch.distributed as dist

from ..data import synthetic
from ..parallel.state import init_distributed
from . import checkpointing
from .timers import Timers
from .trainer import Trainer


def _held_out(batch_of_part, parts, eval_samples: int):
    """The training batch function of `parts[0]`, with `.valid` / `.test` = batch functions of the held-out parts
    (None where --split gives that part no documents)."""
    train = batch_of_part(parts[0], None)
    train.valid = batch_of_part(parts[1], eval_samples) if parts[1] is not None else None
    train.test = batch_of_part(parts[2], eval_samples) if parts[2] is not None else None
    return train


def _split_parts(corpus, num_docs: int, split):
    """[train, validation, test] corpora for --split (documents in file order, contiguous ranges); without --split
    everything trains."""
    if not split:
        return [corpus, None, None]
    from ..data.indexed import split_bounds
    b = split_bounds(split, num_docs)
    assert b[1] > 0, f"--split {split} leaves no training documents out of {num_docs}"
    return [corpus.slice_docs(b[i], b[i + 1]) if b[i + 1] > b[i] else None for i in range(3)]


def make_dataset_batch_fn(trainer: Trainer, prefix: str, train_iters: int, seed: int, eod_token=None, vocab_file=None,
                          split=None, eval_samples: int = 0, titles_prefix=None, data_kw=None):
    """Batches of a GPT token corpus: `prefix`.bin holds the token ids (uint16, or uint32 with `prefix`.u32 present
    instead), `prefix`.npy the document lengths; a Megatron-LM corpus (`prefix`.bin + `prefix`.idx) is read as it
    is.  Batch i is global samples [i * gbs, (i + 1) * gbs) of the
    shuffled sample order (a function of the seed and of --train-iters), so a run resumed with the same
    --train-iters continues where the data stopped."""
    import numpy as np
    if not isinstance(prefix, str) and len(prefix) == 1:
        prefix = prefix[0]
    if trainer.model_name != "gpt":
        assert isinstance(prefix, str), "a blend of several corpora is read for GPT only"
    else:
        assert isinstance(prefix, str) or len(prefix) % 2 == 0, "--data-path: one prefix, or weight prefix pairs"
    if trainer.model_name in ("resnet", "vit"):
        return make_image_batch_fn(trainer, prefix, seed)
    if trainer.model_name == "t5":
        return make_t5_batch_fn(trainer, prefix, train_iters, seed, vocab_file, split=split, eval_samples=eval_samples,
                                data_kw=data_kw)
    if trainer.model_name in ("bert", "ict"):
        special = None
        if vocab_file:      # ids of the special tokens from the WordPiece vocabulary the corpus was encoded with
            from ..data.sentences import SpecialTokens
            from ..tokenizer.wordpiece import load_vocab
            v = load_vocab(vocab_file)
            special = SpecialTokens(cls=v["[CLS]"], sep=v["[SEP]"], mask=v["[MASK]"], pad=v["[PAD]"])
        if trainer.model_name == "ict":
            assert titles_prefix, "the inverse-cloze model with --data-path needs --titles-data-path"
            return make_ict_batch_fn(trainer, prefix, titles_prefix, train_iters, seed, special, split=split,
                                     eval_samples=eval_samples, **{k: v for k, v in (data_kw or {}).items()
                                                                   if k == "query_in_block_prob"})
        return make_bert_batch_fn(trainer, prefix, train_iters, seed, special, split=split, eval_samples=eval_samples,
                                  data_kw=data_kw)
    from ..data.indexed import BlendedDataset, GPTSampleDataset, TokenCorpus
    assert trainer.model_name == "gpt", f"--data-path does not feed the {trainer.model_name} model"
    from ..data import mmap_format

    def load(one: str) -> TokenCorpus:
        if mmap_format.exists(one) and not os.path.exists(one + ".npy"):
            return mmap_format.token_corpus(one)         # a corpus preprocessed for Megatron-LM (<prefix>.idx)
        wide = os.path.exists(one + ".u32")
        return TokenCorpus.from_files(one + (".u32" if wide else ".bin"), one + ".npy",
                                      dtype=np.uint32 if wide else np.uint16)

    # one corpus, or several blended by weight: [w1, prefix1, w2, prefix2, ...]; every corpus is split on its own
    sources = [(1.0, prefix)] if isinstance(prefix, str) else \
        [(float(prefix[k]), prefix[k + 1]) for k in range(0, len(prefix), 2)]
    total_w = sum(w for w, _ in sources)
    assert total_w > 0, "blending weights must not all be zero"
    per_source = []
    for w, one in sources:
        corpus = load(one)
        per_source.append((w / total_w, _split_parts(corpus, len(corpus.sizes), split)))
    parts = []
    for k in range(3):
        have = [(w, p[k]) for w, p in per_source if p[k] is not None]
        parts.append(have or None)
    gbs, seq = trainer.plan["global_batch_size"], trainer.cfg.seq_length

    def batches_of(part, num_samples):
        n = num_samples or train_iters * gbs
        if len(part) == 1:
            data = GPTSampleDataset(part[0][1], seq, num_samples=n, seed=seed)
        else:   # every source a little over its share, so the interleaving never runs one dry (reference:
            # build_train_valid_test_datasets with a blend, runtime/megatron/data/gpt_dataset.py)
            share = sum(w for w, _ in part)
            data = BlendedDataset([GPTSampleDataset(c, seq, num_samples=int(math.ceil(n * w / share * 1.005)), seed=seed)
                                   for w, c in part], [w for w, _ in part], n)

        def batch(i):
            rows = np.stack([data[(i * gbs + j) % len(data)] for j in range(gbs)])
            t = torch.from_numpy(rows)
            out = {"ids": t[:, :-1].contiguous(), "labels": t[:, 1:].contiguous()}
            if eod_token is not None:
                # positions whose INPUT is the end-of-document token would have to predict the first token of an
                # unrelated document: they do not count (reference: eod_mask_loss of
                # get_ltor_masks_and_position_ids, runtime/megatron/utils.py)
                out["loss_mask"] = (out["ids"] != eod_token).to(torch.float32)
            return {k: v.pin_memory() for k, v in out.items()} if torch.cuda.is_available() else out

        return batch

    return _held_out(batches_of, parts, eval_samples)


def _masking_kw(data_kw) -> dict:
    """--mask-prob / --short-seq-prob as the sentence datasets name them; unset flags keep the datasets' defaults."""
    names = {"mask_prob": "masked_lm_prob", "short_seq_prob": "short_seq_prob"}
    return {names[k]: v for k, v in (data_kw or {}).items() if k in names and v is not None}


def make_bert_batch_fn(trainer: Trainer, prefix: str, train_iters: int, seed: int, special=None, split=None,
                       eval_samples: int = 0, data_kw=None):
    """Batches of a sentence corpus written by `data.preprocess --split-sentences`: [CLS] A [SEP] B [SEP] samples with
    masked-LM labels and the sentence-order flag (reference: runtime/megatron/data/bert_dataset.py).  `special`
    names the ids of [CLS], [SEP], [MASK], [PAD]; the default is their place in a BERT WordPiece vocabulary
    (101, 102, 103, 0)."""
    from ..data.preprocess import load_sentence_corpus
    from ..data.sentences import BertDataset, SpecialTokens, bert_batch_of
    tokens = special or SpecialTokens(cls=101, sep=102, mask=103, pad=0)
    cfg, gbs = trainer.cfg, trainer.plan["global_batch_size"]

    def batches_of(part, num_samples):
        data = BertDataset(part, tokens, cfg.vocab, num_samples=num_samples or train_iters * gbs,
                           max_seq_length=cfg.seq_length, seed=seed, binary_head=cfg.binary_head,
                           **_masking_kw(data_kw))
        return lambda i: bert_batch_of(data, range(i * gbs, (i + 1) * gbs))

    corpus = load_sentence_corpus(prefix)
    return _held_out(batches_of, _split_parts(corpus, len(corpus.doc_starts) - 1, split), eval_samples)


def make_ict_batch_fn(trainer: Trainer, prefix: str, titles_prefix: str, train_iters: int, seed: int, special=None,
                      split=None, eval_samples: int = 0, query_in_block_prob: float = 0.1):
    """(query, block) pairs for the inverse-cloze biencoder from two sentence corpora with the same documents in
    the same order: the text (`prefix`) and the titles (`titles_prefix`, all sentences of a document together are
    its title).  A global batch of n sequences holds n / 2 pairs (reference: runtime/megatron/data/ict_dataset.py,
    --titles-data-path and --query-in-block-prob of runtime/megatron/arguments.py)."""
    import numpy as np
    from ..data.indexed import split_bounds
    from ..data.preprocess import load_sentence_corpus
    from ..data.sentences import InverseClozeDataset, SentenceCorpus, SpecialTokens
    from ..models.ict import ict_batch_of
    tokens = special or SpecialTokens(cls=101, sep=102, mask=103, pad=0)
    text, tc = load_sentence_corpus(prefix), load_sentence_corpus(titles_prefix)
    docs = len(text.doc_starts) - 1
    assert len(tc.doc_starts) - 1 == docs, (f"{titles_prefix} holds {len(tc.doc_starts) - 1} documents, "
                                            f"{prefix} holds {docs}: titles and text must pair up")
    titles = [np.asarray(tc.tokens[tc.sent_start[tc.doc_starts[d]]:tc.sent_start[tc.doc_starts[d + 1]]]) for d in range(docs)]
    corpus = SentenceCorpus(text.tokens, text.sizes, text.doc_starts, title_lengths=[len(t) for t in titles])
    cfg, gbs = trainer.cfg, trainer.plan["global_batch_size"]
    assert gbs % 2 == 0, "the inverse-cloze batch holds (query, block) pairs"
    pairs = gbs // 2
    b = split_bounds(split, docs) if split else [0, docs, docs, docs]
    parts = [(corpus.slice_docs(b[k], b[k + 1]), titles[b[k]:b[k + 1]]) if b[k + 1] > b[k] else None for k in range(3)]
    assert parts[0] is not None, f"--split {split} leaves no training documents out of {docs}"

    def batches_of(part, num_samples):
        data = InverseClozeDataset(part[0], part[1], tokens, num_samples=(num_samples or train_iters * gbs) // 2,
                                   max_seq_length=cfg.seq_length, query_in_block_prob=query_in_block_prob, seed=seed)
        return lambda i: ict_batch_of(data, range(i * pairs, (i + 1) * pairs))

    return _held_out(batches_of, parts, eval_samples)


def make_t5_batch_fn(trainer: Trainer, prefix: str, train_iters: int, seed: int, vocab_file: str, extra_ids: int = 100,
                     split=None, eval_samples: int = 0, data_kw=None):
    """Span-corruption batches of a sentence corpus written by `data.preprocess --split-sentences`: masked spans
    become sentinels in the encoder input, the decoder predicts them (reference:
    runtime/megatron/data/t5_dataset.py).  The sentinels, [BOS] and [EOS] are appended to the WordPiece vocabulary,
    so the model's vocabulary has to cover `vocab + 2 + extra_ids` entries."""
    from ..data.preprocess import load_sentence_corpus
    from ..data.sentences import T5Dataset
    from ..tokenizer import build_tokenizer
    assert vocab_file, "T5 with --data-path needs --vocab-file (the WordPiece vocabulary of the corpus)"
    tok = build_tokenizer("BertWordPieceLowerCase", vocab_file, None, vocab_extra_ids=extra_ids)
    cfg, gbs = trainer.cfg, trainer.plan["global_batch_size"]
    assert tok.vocab_size <= cfg.padded_vocab, f"model vocabulary {cfg.padded_vocab} < tokenizer's {tok.vocab_size}"

    def batches_of(part, num_samples):
        from ..data.sentences import t5_batches
        data = T5Dataset(part, tok.special_tokens(), tok.vocab_size, num_samples=num_samples or train_iters * gbs,
                         max_seq_length=cfg.seq_length, max_seq_length_dec=cfg.dec_seq_length, seed=seed,
                         **_masking_kw(data_kw))
        return lambda i: next(t5_batches(data, gbs, 1, start=i * gbs))

    corpus = load_sentence_corpus(prefix)
    return _held_out(batches_of, _split_parts(corpus, len(corpus.doc_starts) - 1, split), eval_samples)


def make_image_batch_fn(trainer: Trainer, root: str, seed: int):
    """Batches of an image folder (`root/train/<class>/<file>`, or `root/<class>/<file>`): random-resized crop, flip,
    colour jitter and the AutoAugment ImageNet policy, each decision a function of (seed, epoch, index) so that a
    resumed run sees the same pictures (reference: runtime/megatron/data/vit_dataset.py:22-42)."""
    from ..data.images import ImageFolder, batch_indices, image_batch
    train_dir = os.path.join(root, "train")
    data = ImageFolder(train_dir if os.path.isdir(train_dir) else root, size=trainer.cfg.image_size, train=True, seed=seed)
    assert len(data.classes) <= trainer.cfg.num_classes, "more class directories than the model has classes"
    gbs = trainer.plan["global_batch_size"]

    def batch(i):
        idx, epoch = batch_indices(len(data), gbs, i, seed)
        return image_batch(data, idx, pin=torch.cuda.is_available(), epoch=epoch)

    batch.valid = batch.test = None
    val_dir = os.path.join(root, "val")
    if os.path.isdir(val_dir):         # held-out pictures: resize + centre crop, in file order
        held = ImageFolder(val_dir, size=trainer.cfg.image_size, train=False, seed=seed)
        batch.valid = lambda i: image_batch(held, [(i * gbs + j) % len(held) for j in range(gbs)],
                                            pin=torch.cuda.is_available())
    return batch


def make_batch_fn(trainer: Trainer):
    plan, cfg = trainer.plan, trainer.cfg
    gbs = plan["global_batch_size"]
    if trainer.model_name == "gpt":
        return lambda i: synthetic.gpt_batch(gbs, cfg.seq_length, cfg.vocab, seed=1234 + i)
    if trainer.model_name == "t5":
        return lambda i: synthetic.t5_batch(gbs, cfg.seq_length, cfg.dec_seq_length, cfg.vocab, seed=1234 + i)
    if trainer.model_name == "bert":
        return lambda i: synthetic.bert_batch(gbs, cfg.seq_length, cfg.vocab, seed=1234 + i)
    if trainer.model_name == "ict":
        def pairs(i):       # synthetic (query, block) pairs: rows 2 k and 2 k + 1 are two views of one token pattern
            b = synthetic.bert_batch(gbs, cfg.seq_length, cfg.vocab, seed=1234 + i)
            ids = b["ids"]
            ids[1::2] = ids[0::2]
            return {"ids": ids, "types": torch.zeros_like(ids), "enc_lens": b["enc_lens"],
                    "labels": torch.arange(gbs // 2).repeat_interleave(2)}
        return pairs
    return lambda i: synthetic.resnet_batch(gbs, cfg.image_size, cfg.num_classes, seed=1234 + i)


class _TerminationRequest:
    """Turns SIGTERM into a flag the training loop reads between iterations (the place of the reference's autoresume
    termination check, runtime/megatron/utils.py:224-242, without its cluster-specific library)."""

    def __init__(self):
        import signal
        self.requested = False
        self._signal = signal
        self._previous = signal.signal(signal.SIGTERM, self._note)

    def _note(self, signum, frame):
        self.requested = True

    def restore(self) -> None:
        self._signal.signal(self._signal.SIGTERM, self._previous)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--flexpipe-config", required=True)
    ap.add_argument("--train-iters", type=int, default=3)
    ap.add_argument("--log-interval", type=int, default=1)
    ap.add_argument("--log-path", default=None)
    ap.add_argument("--lr", type=float, default=1.5e-4)
    ap.add_argument("--min-lr", type=float, default=1.0e-5)
    ap.add_argument("--lr-decay-style", default="cosine", choices=["constant", "linear", "cosine"])
    ap.add_argument("--lr-decay-iters", type=int, default=320000)
    ap.add_argument("--lr-warmup-fraction", type=float, default=0.01)
    ap.add_argument("--weight-decay", type=float, default=0.01)
    ap.add_argument("--clip-grad", type=float, default=1.0)
    ap.add_argument("--optimizer", default="adam", choices=["adam", "sgd"])
    ap.add_argument("--adam-beta1", type=float, default=0.9)
    ap.add_argument("--adam-beta2", type=float, default=0.999)
    ap.add_argument("--adam-eps", type=float, default=1e-8)
    ap.add_argument("--sgd-momentum", type=float, default=0.9)
    ap.add_argument("--lr-warmup-iters", type=int, default=None, help="warm-up iterations (instead of --lr-warmup-fraction)")
    ap.add_argument("--init-method-std", type=float, default=None, help="standard deviation of the weight initialisation")
    ap.add_argument("--log-params-norm", action="store_true", help="L2 norm of the parameters in the iteration line")
    ap.add_argument("--log-num-zeros-in-grad", action="store_true",
                    help="number of zero gradient entries in the iteration line (turns the sharded update off)")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--hidden-dropout", type=float, default=None)
    ap.add_argument("--attention-dropout", type=float, default=None)
    ap.add_argument("--save", default=None)
    ap.add_argument("--load", default=None)
    ap.add_argument("--save-interval", type=int, default=None)
    ap.add_argument("--exit-interval", type=int, default=None)
    ap.add_argument("--exit-duration-in-mins", type=float, default=None,
                    help="save a checkpoint and stop once the run has lasted this long")
    ap.add_argument("--debug-dump", default=None, choices=["output", "grad", "all"],
                    help="with --log-path: per-rank files with statistics of every op's outputs and / or of every "
                         "parameter's weight and gradient, for the first --debug-dump-iters iterations")
    ap.add_argument("--debug-dump-iters", type=int, default=1)
    ap.add_argument("--exit-signal-handler", action="store_true",
                    help="on SIGTERM (a scheduler's notice of preemption) finish the iteration, save a checkpoint "
                         "(with --save) and leave with exit code 0; all ranks leave at the same iteration")
    ap.add_argument("--finetune", action="store_true", help="load the weights only and restart at iteration 0")
    ap.add_argument("--load-resharded", action="store_true",
                    help="the checkpoint under --load was written under ANOTHER plan (other GPU count, tensor-parallel "
                         "degrees or stage split): merge its shards and re-slice the weights for this plan; optimizer "
                         "state is not carried over")
    ap.add_argument("--no-load-optim", action="store_true")
    ap.add_argument("--no-load-rng", action="store_true")
    ap.add_argument("--eval-interval", type=int, default=None, help="evaluate every this many iterations")
    ap.add_argument("--eval-iters", type=int, default=2, help="batches per evaluation")
    ap.add_argument("--tensorboard-dir", default=None, help="scalar logs (written by the last rank)")
    ap.add_argument("--health-check", action="store_true",
                    help="publish a heartbeat every iteration and stop with exit code 3 when a peer failed or went "
                         "silent, instead of waiting in the next collective")
    ap.add_argument("--health-stale-after-s", type=float, default=600.0)
    ap.add_argument("--inject-failure", default=None, metavar="RANK:ITERATION",
                    help="host-side fault injection for tests: that rank raises at the start of that iteration")
    ap.add_argument("--no-fused-comm", action="store_true")
    ap.add_argument("--distribute-checkpointed-activations", action="store_true",
                    help="recomputed segments keep only this rank's 1 / tp share of inputs that the whole "
                         "tensor-parallel group holds, and gather them again in the backward pass")
    ap.add_argument("--deterministic", action="store_true",
                    help="bitwise-reproducible steps: attention backward as the dK/dV + dQ kernel pair instead of the "
                         "fused kernel that sums dQ in arrival order")
    ap.add_argument("--vocab-file", default=None,
                    help="BERT with --data-path: the WordPiece vocabulary of the corpus (ids of [CLS] [SEP] [MASK] [PAD])")
    ap.add_argument("--data-path", default=None, nargs="+",
                    help="corpus prefix (GPT: <prefix>.bin token ids + <prefix>.npy document lengths, or Megatron-LM's "
                         "<prefix>.bin + <prefix>.idx; T5 / BERT: a sentence corpus; Wide-ResNet / ViT: an image "
                         "folder).  GPT also takes a blend: WEIGHT1 PREFIX1 WEIGHT2 PREFIX2 ...  "
                         "Default: synthetic batches")
    ap.add_argument("--num-workers", type=int, default=2,
                    help="with --data-path: threads that prepare the coming batches while the device works (0: "
                         "batches are built in the training loop)")
    ap.add_argument("--mask-prob", type=float, default=None, help="BERT / T5 corpora: share of tokens to mask (0.15)")
    ap.add_argument("--short-seq-prob", type=float, default=None,
                    help="BERT / T5 corpora: share of samples cut to a random shorter length (BERT 0.1, T5 0)")
    ap.add_argument("--query-in-block-prob", type=float, default=None,
                    help="inverse-cloze corpora: how often the query sentence stays inside its block (0.1)")
    ap.add_argument("--titles-data-path", default=None,
                    help="inverse-cloze model: sentence corpus of the documents' titles, same documents in the same "
                         "order as --data-path")
    ap.add_argument("--split", default=None, metavar="TRAIN,VALID,TEST",
                    help="with --data-path: weights of the training / validation / test parts of the corpus (whole "
                         "documents, in file order), e.g. 949,50,1; --eval-interval then evaluates on the validation "
                         "part and the end of training on the test part.  Default: everything trains and evaluation "
                         "draws from the same corpus.  An image folder holds its validation part in <root>/val")
    ap.add_argument("--eod-mask-loss", type=int, default=None, metavar="EOD_TOKEN_ID",
                    help="with --data-path: positions whose input is this end-of-document token do not count in the loss")
    ap.add_argument("--interleave-factor", type=int, default=1,
                    help="model chunks per pipeline stage (interleaved 1F1B); re-cuts the plan's stages evenly")
    ap.add_argument("--interleave-ops", type=int, nargs="+", default=None,
                    help="ops of every virtual stage (stages x interleave-factor numbers) instead of the even cut")
    ap.add_argument("--distributed-backend", default=None, choices=[None, "nccl", "gloo"])
    # launch scripts written for the reference pass many Megatron flags the plan JSON already determines (--fp16,
    # --num-layers, --micro-batch-size ...): they are accepted and reported, not refused
    args, ignored = ap.parse_known_args(argv)
    rank, world, _ = init_distributed(args.distributed_backend)
    if ignored and rank == 0:
        print("flags without effect here (the plan and the defaults decide): " + " ".join(ignored), flush=True)
    with open(args.flexpipe_config) as f:
        plan = json.load(f)
    if args.interleave_factor > 1:
        from .schedules import interleave_plan
        plan = interleave_plan(plan, args.interleave_factor, args.interleave_ops)
    if args.deterministic:
        from ..ops import functional as F
        F.set_deterministic(True)
    overrides = {}
    if args.hidden_dropout is not None:
        overrides["hidden_dropout"] = args.hidden_dropout
    if args.attention_dropout is not None:
        overrides["attention_dropout"] = args.attention_dropout
    if args.init_method_std is not None:
        overrides["init_std"] = args.init_method_std
    warmup = args.lr_warmup_iters if args.lr_warmup_iters is not None else int(args.lr_warmup_fraction * args.lr_decay_iters)
    trainer = Trainer(plan, model_overrides=overrides, rank=rank, world_size=world, seed=args.seed, lr=args.lr, min_lr=args.min_lr,
                      weight_decay=args.weight_decay, clip_grad=args.clip_grad, lr_decay_steps=args.lr_decay_iters,
                      lr_warmup_steps=warmup, lr_style=args.lr_decay_style,
                      optimizer=args.optimizer, fused_comm=not args.no_fused_comm,
                      adam_betas=(args.adam_beta1, args.adam_beta2), adam_eps=args.adam_eps,
                      sgd_momentum=args.sgd_momentum, shard_optimizer=not args.log_num_zeros_in_grad,
                      distribute_checkpointed_activations=args.distribute_checkpointed_activations)
    if args.load and args.load_resharded:
        trainer.iteration = 0 if args.finetune else checkpointing.load_under_plan(trainer, args.load)
        trainer.lr_schedule.step(trainer.iteration)      # the schedule continues where the old run stopped
    elif args.load:
        checkpointing.load_checkpoint(trainer, args.load, load_optim=not args.no_load_optim,
                                      load_rng=not args.no_load_rng, finetune=args.finetune)
    monitor = None
    if args.health_check and world > 1:
        from .health import HealthMonitor, store_from_env
        monitor = HealthMonitor(store_from_env(rank, world), rank, world, stale_after_s=args.health_stale_after_s)
        trainer.health_monitor = monitor     # a device status error is published to the peers before it is raised
    fail_rank, fail_iter = (int(x) for x in args.inject_failure.split(":")) if args.inject_failure else (-1, -1)
    writer = None
    if args.tensorboard_dir and rank == world - 1:
        from torch.utils.tensorboard import SummaryWriter
        writer = SummaryWriter(log_dir=args.tensorboard_dir)
    t_start = time.time()
    gbs = plan["global_batch_size"]
    eval_rounds = args.train_iters // args.eval_interval + 1 if args.eval_interval else 1
    batch_fn = (make_dataset_batch_fn(trainer, args.data_path, args.train_iters, args.seed, args.eod_mask_loss,
                                      args.vocab_file, split=args.split,
                                      eval_samples=max(1, eval_rounds * args.eval_iters) * gbs,
                                      titles_prefix=args.titles_data_path,
                                      data_kw={k: v for k, v in dict(mask_prob=args.mask_prob,
                                                                      short_seq_prob=args.short_seq_prob,
                                                                      query_in_block_prob=args.query_in_block_prob).items()
                                               if v is not None})
                if args.data_path
                else make_batch_fn(trainer))
    if args.data_path and args.num_workers > 0:
        from ..data.prefetch import Prefetcher
        batch_fn = Prefetcher(batch_fn, workers=args.num_workers, stop=args.train_iters)
    # synthetic batches are generated on the host before the loop (a pool of up to 4, reused in turn): building
    # a 768-image batch takes longer than a training step and is not part of what an iteration measures
    # batch of iteration `it` is batch_fn(it % 4) whether the run is fresh or resumed, so a resumed run sees the
    # batches the uninterrupted run would have seen
    pool = {} if args.data_path else \
        {i % 4: batch_fn(i % 4) for i in range(trainer.iteration, min(args.train_iters, trainer.iteration + 4))}
    timers = Timers(trainer.device.type == "cuda")
    config_name = os.path.splitext(os.path.basename(args.flexpipe_config))[0]
    regions = ["iteration", "forward-backward", "backward-params-all-reduce", "optimizer"]
    extra = {}             # further columns of the iteration line
    dump = None
    if args.debug_dump:
        assert args.log_path, "--debug-dump writes under --log-path"
        from .debug_dump import DebugDump
        dump = DebugDump(trainer, args.log_path, config_name, args.debug_dump, args.debug_dump_iters)
    term = _TerminationRequest() if args.exit_signal_handler else None

    def one_step(it):
        timers("iteration").start()
        batch = trainer.to_device(batch_fn(it) if args.data_path else pool[it % 4])
        timers("forward-backward").start()
        loss = trainer.forward_backward(batch)
        trainer._fold_autograd_grads()
        timers("forward-backward").stop()
        timers("backward-params-all-reduce").start()
        if dump is not None:
            dump.gradients("before the reduction")
        trainer.optimizer.reduce_gradients()
        if trainer._tied is not None:
            trainer._tied.sync_grads()
        timers("backward-params-all-reduce").stop()
        if dump is not None:
            dump.gradients("after the reduction and the tied-weight sync")
        if args.log_num_zeros_in_grad and (it + 1) % args.log_interval == 0:
            extra["num zeros"] = trainer.optimizer.count_zeros_in_grad()
        timers("optimizer").start()
        lr = trainer.lr_schedule.get_lr()
        trainer.optimizer.step(lr=lr)
        trainer.lr_schedule.step()
        trainer.iteration += 1
        timers("optimizer").stop()
        timers("iteration").stop()
        return loss, lr

    for it in range(trainer.iteration, args.train_iters):
        if monitor is not None:
            from .health import PeerFailure
            try:
                monitor.beat(it)            # a failed or silent peer ends the run HERE, before the next collective
            except PeerFailure as e:
                print(f"rank {rank}: stopping before iteration {it + 1}: {e}", flush=True)
                sys.stdout.flush()
                os._exit(3)                 # no collective clean-up: the peer it would wait for is gone
        with (monitor.guard() if monitor is not None else contextlib.nullcontext()):
            if rank == fail_rank and it == fail_iter:
                raise RuntimeError(f"injected failure at iteration {it}")
            loss, lr = one_step(it)
        if (it + 1) % args.log_interval == 0:
            row = timers.row(regions)
            lv = trainer.loss_value({"loss_tensor": loss})
            mem = torch.cuda.max_memory_allocated() / 2 ** 20 if trainer.device.type == "cuda" else 0.0
            if args.log_params_norm:
                extra["params norm"] = trainer.optimizer.params_norm()
            if trainer.optimizer.skipped_steps():
                extra["number of skipped iterations"] = trainer.optimizer.skipped_steps()
            more = "".join(f" | {k}: {v:.3f}" if isinstance(v, float) else f" | {k}: {v}" for k, v in extra.items())
            if rank == world - 1:
                print(f" iteration {it + 1:8d}/{args.train_iters:8d} | consumed samples: "
                      f"{(it + 1) * plan['global_batch_size']:12d} | elapsed time per iteration (ms): "
                      f"{row['iteration']:.1f} | learning rate: {lr:.3E} | global batch size: "
                      f"{plan['global_batch_size']:5d} | lm loss: {lv:.6E} | grad norm: {trainer.optimizer.grad_norm():.3f}"
                      + more, flush=True)
            if writer is not None:
                writer.add_scalar("learning-rate", lr, it + 1)
                writer.add_scalar("lm loss", lv, it + 1)
                writer.add_scalar("grad-norm", trainer.optimizer.grad_norm(), it + 1)
                for k, v in extra.items():
                    writer.add_scalar(k.replace(" ", "-"), v, it + 1)
                writer.add_scalar("samples per second", plan["global_batch_size"] / (row["iteration"] / 1e3), it + 1)
                for r in regions:
                    writer.add_scalar(f"{r}-time", row[r], it + 1)
            if it == args.train_iters - 1 and args.log_path:
                os.makedirs(os.path.join(args.log_path, "csv"), exist_ok=True)
                path = os.path.join(args.log_path, "csv", f"{config_name}_stage{trainer.pstate.stage}_rank{rank}.csv")
                with open(path, "w", newline="") as f:
                    w = csv.writer(f)
                    w.writerow(["global_batch_size", "time"] + regions[1:] + ["max_allocated_memory(MB)"])
                    w.writerow([plan["global_batch_size"], f"{row['iteration']:.2f}"] +
                               [f"{row[r]:.2f}" for r in regions[1:]] + [f"{mem:.0f}"])
        if args.save and args.save_interval and (it + 1) % args.save_interval == 0:
            checkpointing.save_checkpoint(trainer, args.save)
        if args.eval_interval and (it + 1) % args.eval_interval == 0:
            held = getattr(batch_fn, "valid", None)
            if held is not None:           # the validation part, continued from where the last evaluation stopped
                first = ((it + 1) // args.eval_interval - 1) * args.eval_iters
                ev = trainer.evaluate(held(first + j) for j in range(args.eval_iters))
            else:
                direct = getattr(batch_fn, "fn", batch_fn)        # not through the prefetcher: out of its sequence
                ev = trainer.evaluate(direct(10 ** 6 + it * args.eval_iters + j) for j in range(args.eval_iters))
            if rank == world - 1:
                print(f" validation loss at iteration {it + 1} | " +
                      " | ".join(f"{k} value: {v:.6E}" for k, v in ev.items()), flush=True)
            if writer is not None:
                for k, v in ev.items():
                    writer.add_scalar(f"{k} validation", v, it + 1)
        if args.exit_interval and (it + 1) % args.exit_interval == 0:
            break
        if args.exit_duration_in_mins is not None:
            # every rank must take the same decision: the slowest clock decides
            over = torch.tensor([float((time.time() - t_start) / 60.0 > args.exit_duration_in_mins)],
                                device=trainer.device)
            if world > 1:
                dist.all_reduce(over, op=dist.ReduceOp.MAX)
            if over.item() > 0:
                if rank == 0:
                    print(f"exiting after {(time.time() - t_start) / 60.0:.1f} minutes at iteration {it + 1}", flush=True)
                break
        if term is not None:
            # a rank that got the signal tells the others: they all stop after the same iteration
            asked = torch.tensor([float(term.requested)], device=trainer.device)
            if world > 1:
                dist.all_reduce(asked, op=dist.ReduceOp.MAX)
            if asked.item() > 0:
                if rank == 0:
                    print(f"termination requested: stopping after iteration {it + 1}", flush=True)
                break
    if term is not None:
        term.restore()
    if dump is not None:
        dump.close()
    if args.save:
        checkpointing.save_checkpoint(trainer, args.save)
    held = getattr(batch_fn, "test", None)
    if held is not None and args.eval_iters > 0:
        ev = trainer.evaluate(held(j) for j in range(args.eval_iters))
        if rank == world - 1:
            print(" test loss at the end of training | " + " | ".join(f"{k} value: {v:.6E}" for k, v in ev.items()),
                  flush=True)
    if writer is not None:
        writer.close()
    if hasattr(batch_fn, "close"):
        batch_fn.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
