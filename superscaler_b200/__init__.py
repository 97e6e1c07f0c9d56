"""superscaler_b200: a Blackwell (sm_100a) native automatic-parallelism training framework.

Workflow (same three steps as the Aceso artifact of microsoft/SuperScaler): profile the ops and
collectives on the target GPUs (`superscaler_b200.profiler`), search a per-op TP / DP / PP / recompute
plan on CPU (`superscaler_b200.search`), and train from the plan JSON (`superscaler_b200.runtime`).
"""
__version__ = "0.1.0"
