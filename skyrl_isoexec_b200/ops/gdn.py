def gdn_block(y, model, i, fc, kv_idx):
    raise NotImplementedError("GDN block is provided by ops/gdn.py")
