"""Text generation with a GPT plan: temperature / top-k / top-p (nucleus) sampling or greedy decoding.

Counterpart of the reference's sampling utilities (runtime/megatron/text_generation_utils.py: top_k_logits,
sample_sequence_batch, generate_samples_*).  The op-list model has no key / value cache (neither have the
reference's flex ops), so every new token re-runs the causal forward over the whole window of `seq_length`
positions: prompts are right-padded, and because attention is causal the padding cannot influence the position
that is read.  Runs every plan `Trainer.logits` runs (one GPU, tensor / data parallel groups, pipelines); every rank
calls generate with the same arguments and seed and returns the same sequences.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


def filter_logits(logits: torch.Tensor, top_k: int = 0, top_p: float = 0.0) -> torch.Tensor:
    """Sets to -inf every logit outside the k largest and outside the smallest set whose probability mass
    reaches top_p (the most likely token always survives).  logits: [batch, vocab]."""
    out = logits.clone()
    if top_k > 0:
        kth = torch.topk(out, min(top_k, out.shape[-1]), dim=-1).values[..., -1:]
        out[out < kth] = float("-inf")
    if top_p > 0.0:
        sorted_logits, order = torch.sort(out, dim=-1, descending=True)
        mass = torch.softmax(sorted_logits, dim=-1).cumsum(dim=-1)
        drop = mass - torch.softmax(sorted_logits, dim=-1) >= top_p     # mass BEFORE this token already enough
        drop[..., 0] = False
        sorted_logits[drop] = float("-inf")
        out = torch.full_like(out, float("-inf")).scatter(-1, order, sorted_logits)
    return out


def sample_next(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0,
                greedy: bool = False, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """One token id per row of logits [batch, vocab]."""
    logits = logits.float()
    if greedy or temperature == 0.0:
        return logits.argmax(dim=-1)
    probs = torch.softmax(filter_logits(logits / temperature, top_k, top_p), dim=-1)
    return torch.multinomial(probs, 1, generator=generator).squeeze(-1)


@torch.no_grad()
def generate(trainer, prompts: Sequence[Sequence[int]], max_new_tokens: int, eod: Optional[int] = None,
             temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0, greedy: bool = False, seed: int = 1234,
             vocab_size: Optional[int] = None, pad: int = 0) -> List[List[int]]:
    """Continues every prompt by up to max_new_tokens tokens (stops a sequence at `eod`).  `vocab_size` cuts the
    padded part of the vocabulary off before sampling.  Returns prompt + continuation per sequence."""
    S = trainer.cfg.seq_length
    seqs = [list(map(int, p)) for p in prompts]
    assert all(0 < len(p) < S for p in seqs), "prompts must be non-empty and shorter than the model's window"
    done = [False] * len(seqs)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    for _ in range(max_new_tokens):
        active = [i for i, d in enumerate(done) if not d and len(seqs[i]) < S]
        if not active:
            break
        ids = torch.full((len(seqs), S), pad, dtype=torch.int64)
        for i, s in enumerate(seqs):
            ids[i, : min(len(s), S)] = torch.tensor(s[:S])
        logits = trainer.logits(ids)
        last = torch.stack([logits[i, min(len(seqs[i]), S) - 1] for i in range(len(seqs))]).float().cpu()
        if vocab_size is not None:
            last = last[:, :vocab_size]
        nxt = sample_next(last, temperature, top_k, top_p, greedy, gen).tolist()
        for i in active:
            seqs[i].append(int(nxt[i]))
            if eod is not None and nxt[i] == eod:
                done[i] = True
    return seqs


def generate_text(trainer, tokenizer, texts: Sequence[str], max_new_tokens: int, **kw) -> List[str]:
    """Tokenize, generate, detokenize (the continuation stops at the tokenizer's end-of-document id)."""
    eod = getattr(tokenizer, "eod", None)
    out = generate(trainer, [tokenizer.tokenize(t) for t in texts], max_new_tokens, eod=eod,
                   vocab_size=tokenizer.vocab_size, **kw)
    return [tokenizer.detokenize([i for i in s if i != eod]) for s in out]


def main(argv=None) -> None:
    """Command line (counterpart of the reference's tools/generate_samples_gpt.py + runtime/megatron/
    text_generation_utils.py: generate_samples_input_from_file / generate_and_write_samples_unconditional):

        python [-m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1] \\
            -m superscaler_b200.runtime.generation --flexpipe-config plan.json --load ckpt/ \\
            --vocab-file vocab.json --merge-file merges.txt --prompt "The capital of France is" \\
            [--sample-input-file prompts.txt] [--sample-output-file out.txt] [--num-samples 4] \\
            --out-seq-length 64 [--greedy | --temperature 0.9 --top_k 40 --top_p 0.9]

    Prompts come from --prompt (repeatable), from the lines of --sample-input-file, or -- with --num-samples alone
    -- are the end-of-document token (unconditional samples).  The checkpoint may have been written under another
    plan of the same model.  Rank 0 prints (and writes) the texts."""
    import argparse
    import json

    from ..parallel.state import init_distributed
    from ..tokenizer import build_tokenizer
    from . import checkpointing
    from .trainer import Trainer
    ap = argparse.ArgumentParser(description=main.__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--flexpipe-config", required=True)
    ap.add_argument("--load", default=None, help="checkpoint directory (default: random weights)")
    ap.add_argument("--tokenizer-type", default="GPT2BPETokenizer")
    ap.add_argument("--vocab-file", required=True)
    ap.add_argument("--merge-file", default=None)
    ap.add_argument("--prompt", action="append", default=[])
    ap.add_argument("--sample-input-file", default=None)
    ap.add_argument("--sample-output-file", default=None)
    ap.add_argument("--num-samples", type=int, default=0, help="unconditional samples when no prompt is given")
    ap.add_argument("--out-seq-length", type=int, default=64, help="new tokens per sample")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top_k", "--top-k", type=int, default=0)
    ap.add_argument("--top_p", "--top-p", type=float, default=0.0)
    ap.add_argument("--greedy", action="store_true")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--distributed-backend", default=None, choices=[None, "nccl", "gloo"])
    args, _ = ap.parse_known_args(argv)
    rank, world, _ = init_distributed(args.distributed_backend)
    with open(args.flexpipe_config) as f:
        plan = json.load(f)
    trainer = Trainer(plan, rank=rank, world_size=world, seed=args.seed,
                      model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0))
    if args.load:
        checkpointing.load_under_plan(trainer, args.load)
    tok = build_tokenizer(args.tokenizer_type, args.vocab_file, args.merge_file)
    assert tok.vocab_size <= trainer.cfg.padded_vocab, "the tokenizer has more entries than the model's embedding table"
    texts = list(args.prompt)
    if args.sample_input_file:
        with open(args.sample_input_file) as f:
            texts += [line.rstrip("\n") for line in f if line.strip()]
    kw = dict(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, greedy=args.greedy, seed=args.seed)
    if texts:
        outs = generate_text(trainer, tok, texts, args.out_seq_length, **kw)
    else:
        assert args.num_samples > 0, "give --prompt, --sample-input-file or --num-samples"
        seqs = generate(trainer, [[tok.eod]] * args.num_samples, args.out_seq_length, eod=None,
                        vocab_size=tok.vocab_size, **kw)
        outs = [tok.detokenize([i for i in s[1:] if i != tok.eod]) for s in seqs]
    if rank == 0:
        for i, o in enumerate(outs):
            print(f"--- sample {i} ---\n{o}", flush=True)
        if args.sample_output_file:
            with open(args.sample_output_file, "w") as f:
                f.write(json.dumps(outs, indent=1))


if __name__ == "__main__":
    main()
