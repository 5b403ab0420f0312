def moe_block(y, model, i):
    raise NotImplementedError("MoE block is provided by ops/moe.py")
