"""Shared builders for tiny plans used by the tests."""
from superscaler_b200.models.gpt import gpt_op_names


def tiny_gpt_plan(layers=2, seq=128, hidden=128, heads=2, head_dim=64, vocab=512, global_bs=4, micro_bs=2,
                  recompute=0, num_gpus=(1,), ops_per_stage=None, tp=None, dp=None):
    names = gpt_op_names(layers)
    n = len(names)
    stages = len(num_gpus)
    if ops_per_stage is None:
        per = n // stages
        ops_per_stage = [per] * stages
        ops_per_stage[-1] += n - per * stages
    tp = tp or [1] * stages
    dp = dp or [g // t for g, t in zip(num_gpus, tp)]
    rc_flat = [0] + [recompute] * (n - 3) + [0, 0]
    rc, start = [], 0
    for c in ops_per_stage:
        rc.append(rc_flat[start:start + c])
        start += c
    return {"model_name": "gpt", "model_size": "tiny", "num_layers": layers, "seq_length": seq,
            "max_position_embeddings": seq, "num_attention_heads": heads, "hidden_size": hidden,
            "kv_channels": head_dim, "vocab_size": vocab, "global_batch_size": global_bs,
            "micro_batch_size": micro_bs, "num_stages": stages, "num_gpus": list(num_gpus),
            "checkpoint_activations": [bool(recompute)] * stages, "resharding_stages": [False] * stages,
            "num_ops_in_each_stage": list(ops_per_stage),
            "model_parallel_size_of_each_op": [[tp[s]] * ops_per_stage[s] for s in range(stages)],
            "data_parallel_size_of_each_op": [[dp[s]] * ops_per_stage[s] for s in range(stages)],
            "recompute_ops": rc, "algo_of_each_op": [[0] * c for c in ops_per_stage]}


def tiny_t5_plan(layers=1, enc_seq=64, dec_seq=32, hidden=64, heads=2, head_dim=32, ffn=128, vocab=256, global_bs=4,
                 micro_bs=2, recompute=0, num_gpus=(1,), ops_per_stage=None, tp=None):
    from superscaler_b200.models.t5 import t5_op_names
    names = t5_op_names(layers)
    n = len(names)
    stages = len(num_gpus)
    if ops_per_stage is None:
        per = n // stages
        ops_per_stage = [per] * stages
        ops_per_stage[-1] += n - per * stages
    tp = tp or [1] * stages
    dp = [g // t for g, t in zip(num_gpus, tp)]
    never = ("encoder-embedding", "decoder-embedding", "t5-post-process")
    rc_flat = [0 if nm in never else recompute for nm in names]
    rc, start = [], 0
    for c in ops_per_stage:
        rc.append(rc_flat[start:start + c])
        start += c
    return {"model_name": "t5", "model_size": "tiny", "num_layers": layers, "encoder_seq_length": enc_seq,
            "decoder_seq_length": dec_seq, "max_position_embeddings": enc_seq, "num_attention_heads": heads,
            "kv_channels": head_dim, "hidden_size": hidden, "ffn_hidden_size": ffn, "vocab_size": vocab,
            "global_batch_size": global_bs, "micro_batch_size": micro_bs, "num_stages": stages,
            "num_gpus": list(num_gpus), "checkpoint_activations": [bool(recompute)] * stages,
            "resharding_stages": [False] * stages, "num_ops_in_each_stage": list(ops_per_stage),
            "model_parallel_size_of_each_op": [[tp[s]] * ops_per_stage[s] for s in range(stages)],
            "data_parallel_size_of_each_op": [[dp[s]] * ops_per_stage[s] for s in range(stages)],
            "recompute_ops": rc, "algo_of_each_op": [[0] * c for c in ops_per_stage]}


def tiny_resnet_plan(blocks=(1, 1, 1, 1), in_channels=8, width_factor=2, global_bs=4, micro_bs=2, recompute=0,
                     num_gpus=(1,), ops_per_stage=None, tp=None):
    n = 4 + 8 * sum(blocks) + 2
    stages = len(num_gpus)
    if ops_per_stage is None:
        per = n // stages
        ops_per_stage = [per] * stages
        ops_per_stage[-1] += n - per * stages
    tp = tp or [1] * stages
    dp = [g // t for g, t in zip(num_gpus, tp)]
    rc_flat = [0] + [recompute] * (n - 2) + [0]
    rc, start = [], 0
    for c in ops_per_stage:
        rc.append(rc_flat[start:start + c])
        start += c
    return {"model_name": "resnet", "model_size": "tiny", "num_layers": list(blocks), "in_channels": in_channels,
            "width_factor": width_factor, "global_batch_size": global_bs, "micro_batch_size": micro_bs,
            "num_stages": stages, "num_gpus": list(num_gpus), "checkpoint_activations": [bool(recompute)] * stages,
            "resharding_stages": [False] * stages, "num_ops_in_each_stage": list(ops_per_stage),
            "model_parallel_size_of_each_op": [[tp[s]] * ops_per_stage[s] for s in range(stages)],
            "data_parallel_size_of_each_op": [[dp[s]] * ops_per_stage[s] for s in range(stages)],
            "recompute_ops": rc, "algo_of_each_op": [[0] * c for c in ops_per_stage]}


def tiny_bert_plan(**kw):
    """The GPT helper's plan with the BERT op list (same op count: embedding + 13 per layer + final LayerNorm + head)."""
    plan = tiny_gpt_plan(**kw)
    plan["model_name"] = "bert"
    return plan


def tiny_vit_plan(image_size=32, patch=8, num_classes=10, **kw):
    """The GPT helper's plan with the ViT op list (same op count); seq / vocab arguments of the helper are unused."""
    plan = tiny_gpt_plan(**kw)
    plan.update(model_name="vit", image_size=image_size, patch_dim=patch, num_classes=num_classes)
    return plan


def tiny_ict_plan(projection=16, **kw):
    plan = tiny_gpt_plan(**kw)
    plan.update(model_name="ict", biencoder_projection_dim=projection)
    return plan
