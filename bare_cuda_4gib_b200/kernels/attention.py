"""Launcher of the tensor-core paged attention (filled in with the fast kernel)."""


def plan_for(head_dim, heads, kv_heads):
    return None
