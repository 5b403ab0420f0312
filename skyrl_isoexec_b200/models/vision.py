"""Vision tower for vision-language policies: image patches -> rows of the decoder's embedding space, spliced into the
token stream at the image placeholder tokens (reference: the multimodal path of R/backends/skyrl_train/workers/
model_wrapper.py:250-330, which hands ``pixel_values`` / ``image_grid_thw`` to a Hugging Face VLM; here the tower is
this framework's own).

Input format (the one Qwen2-VL style processors emit, so data prepared for the reference reads here):

* ``pixel_values``    ``[n_patches, C * patch * patch]``: flattened patches of all images of a sequence, image after image;
  within an image the patches of one ``merge x merge`` neighbourhood are consecutive (row-major over neighbourhoods,
  row-major inside one);
* ``image_grid_thw``  ``[n_images, 3]``: (frames = 1, patch rows, patch columns) per image; rows and columns are multiples of
  ``merge``.

An image of ``h x w`` patches becomes ``h * w / merge**2`` rows, one per placeholder token (``num_image_tokens``).

Architecture: linear patch embedding + learned row and column position embeddings, pre-LayerNorm transformer blocks with
bidirectional attention over the patches of ONE image and a GELU MLP, then LayerNorm, concatenation of every
``merge x merge`` neighbourhood and a two-layer projector to the decoder's hidden size.

The tower is FROZEN and runs without gradient on both sides of the rollout / training boundary. Each image is processed
on its own, so a given image always meets the same shapes and the same library kernels: its feature rows are the same
bits in the engine and in the trainer, and to the decoder they are input data like token embeddings. (Its matmuls are
library calls, not this framework's kernels; it is a few percent of a step.) Its weights come from the seed, or from a
``visual.*`` state dict (``load_state_dict``); they are not part of the trainer's flat parameter buffer, the optimizer
or the checkpoints.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as tnf


class VisionTower:
    def __init__(self, cfg, device, seed: int = 0):
        """``cfg``: a ModelConfig with ``vision_depth > 0``."""
        assert cfg.vision_depth > 0 and cfg.image_token_id >= 0
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = cfg.torch_dtype
        self.patch, self.merge = cfg.vision_patch, cfg.vision_merge
        self.h, self.heads = cfg.vision_hidden, cfg.vision_heads
        self.in_dim = 3 * self.patch * self.patch
        g = torch.Generator().manual_seed(seed + 7717)
        H, Dout, m2 = self.h, cfg.hidden_size, self.merge * self.merge

        def w(*shape, fan_in):
            return (torch.randn(*shape, generator=g) / math.sqrt(fan_in)).to(self.dtype).to(self.device)

        z = lambda *s: torch.zeros(*s, dtype=self.dtype, device=self.device)
        o = lambda *s: torch.ones(*s, dtype=self.dtype, device=self.device)
        self.w: dict[str, torch.Tensor] = {
            "visual.patch_embed.weight": w(H, self.in_dim, fan_in=self.in_dim), "visual.patch_embed.bias": z(H),
            "visual.pos_row": w(cfg.vision_max_grid, H, fan_in=H) * 0.5, "visual.pos_col": w(cfg.vision_max_grid, H, fan_in=H) * 0.5,
            "visual.merger.ln.weight": o(H), "visual.merger.ln.bias": z(H),
            "visual.merger.fc1.weight": w(m2 * H, m2 * H, fan_in=m2 * H), "visual.merger.fc1.bias": z(m2 * H),
            "visual.merger.fc2.weight": w(Dout, m2 * H, fan_in=m2 * H), "visual.merger.fc2.bias": z(Dout),
        }
        for i in range(cfg.vision_depth):
            p = f"visual.blocks.{i}."
            self.w.update({
                p + "ln1.weight": o(H), p + "ln1.bias": z(H), p + "ln2.weight": o(H), p + "ln2.bias": z(H),
                p + "qkv.weight": w(3 * H, H, fan_in=H), p + "qkv.bias": z(3 * H),
                p + "proj.weight": w(H, H, fan_in=H), p + "proj.bias": z(H),
                p + "fc1.weight": w(4 * H, H, fan_in=H), p + "fc1.bias": z(4 * H),
                p + "fc2.weight": w(H, 4 * H, fan_in=4 * H), p + "fc2.bias": z(H),
            })

    # ------------------------------------------------------------------ weights
    def state_dict(self) -> dict:
        return {k: v.detach().cpu().clone() for k, v in self.w.items()}

    def load_state_dict(self, sd: dict) -> None:
        for k, v in self.w.items():
            if k not in sd:
                raise KeyError(f"vision weights lack {k}")
            if tuple(sd[k].shape) != tuple(v.shape):
                raise ValueError(f"{k}: shape {tuple(sd[k].shape)} in the file, {tuple(v.shape)} in the model")
            v.copy_(sd[k].to(v.dtype))

    def to(self, device) -> "VisionTower":
        self.device = torch.device(device)
        self.w = {k: v.to(self.device) for k, v in self.w.items()}
        return self

    # ------------------------------------------------------------------ shapes
    def num_image_tokens(self, grid) -> int:
        """Placeholder tokens of one image with grid (t, h, w)."""
        t, h, w = (int(x) for x in grid)
        return t * h * w // (self.merge * self.merge)

    def _positions(self, h: int, w: int):
        """Row and column index of every patch in the merge-neighbourhood order of ``pixel_values``."""
        m = self.merge
        r = torch.arange(h).view(h // m, m, 1, 1).expand(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
        c = torch.arange(w).view(1, 1, w // m, m).expand(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
        return r.to(self.device), c.to(self.device)

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def encode_image(self, patches: torch.Tensor, grid) -> torch.Tensor:
        """``patches`` [h * w, C * patch * patch] of one image -> [h * w / merge**2, hidden_size of the decoder]."""
        t, h, w = (int(x) for x in grid)
        if t != 1:
            raise ValueError("video inputs (more than one frame per grid entry) are not supported")
        if h % self.merge or w % self.merge or max(h, w) > self.cfg.vision_max_grid:
            raise ValueError(f"image grid {h} x {w} must be multiples of {self.merge} and at most {self.cfg.vision_max_grid}")
        if patches.shape != (h * w, self.in_dim):
            raise ValueError(f"pixel_values of shape {tuple(patches.shape)} do not match a grid of {h} x {w} patches of {self.in_dim} values")
        W = self.w
        x = tnf.linear(patches.to(self.device, self.dtype), W["visual.patch_embed.weight"], W["visual.patch_embed.bias"])
        r, c = self._positions(h, w)
        x = x + W["visual.pos_row"][r] + W["visual.pos_col"][c]
        N, H, nh = x.shape[0], self.h, self.heads
        for i in range(self.cfg.vision_depth):
            p = f"visual.blocks.{i}."
            y = tnf.layer_norm(x, (H,), W[p + "ln1.weight"], W[p + "ln1.bias"], 1e-6)
            qkv = tnf.linear(y, W[p + "qkv.weight"], W[p + "qkv.bias"]).view(N, 3, nh, H // nh).permute(1, 2, 0, 3)
            a = tnf.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])            # [heads, N, d], every patch sees every patch
            x = x + tnf.linear(a.permute(1, 0, 2).reshape(N, H), W[p + "proj.weight"], W[p + "proj.bias"])
            y = tnf.layer_norm(x, (H,), W[p + "ln2.weight"], W[p + "ln2.bias"], 1e-6)
            x = x + tnf.linear(tnf.gelu(tnf.linear(y, W[p + "fc1.weight"], W[p + "fc1.bias"])), W[p + "fc2.weight"], W[p + "fc2.bias"])
        x = tnf.layer_norm(x, (H,), W["visual.merger.ln.weight"], W["visual.merger.ln.bias"], 1e-6)
        x = x.view(N // (self.merge ** 2), self.merge ** 2 * H)                       # neighbours are consecutive rows
        x = tnf.gelu(tnf.linear(x, W["visual.merger.fc1.weight"], W["visual.merger.fc1.bias"]))
        return tnf.linear(x, W["visual.merger.fc2.weight"], W["visual.merger.fc2.bias"])

    @torch.no_grad()
    def encode(self, pixel_values: torch.Tensor, image_grid_thw: torch.Tensor) -> torch.Tensor:
        """All images of one sequence, image by image: [sum of placeholder tokens, hidden_size]."""
        grids = image_grid_thw.view(-1, 3).tolist()
        out, lo = [], 0
        for g in grids:
            n = int(g[0]) * int(g[1]) * int(g[2])
            out.append(self.encode_image(pixel_values[lo:lo + n], g))
            lo += n
        if lo != pixel_values.shape[0]:
            raise ValueError(f"pixel_values has {pixel_values.shape[0]} patches, image_grid_thw accounts for {lo}")
        return torch.cat(out, 0) if out else torch.zeros(0, self.cfg.hidden_size, dtype=self.dtype, device=self.device)


def patchify(image: torch.Tensor, patch: int = 14, merge: int = 2, mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5)):
    """One image ``[3, H, W]`` (uint8 0..255 or float 0..1) -> (pixel_values [h * w, 3 * patch * patch] float32, grid
    tensor [1, 3]). Height and width are cropped down to multiples of ``patch * merge``. Patches come out in the
    merge-neighbourhood order the tower expects."""
    if image.dim() != 3 or image.shape[0] != 3:
        raise ValueError(f"an image is [3, H, W], got {tuple(image.shape)}")
    x = image.float() / 255.0 if image.dtype == torch.uint8 else image.float()
    unit = patch * merge
    Hh, Ww = (x.shape[1] // unit) * unit, (x.shape[2] // unit) * unit
    if Hh == 0 or Ww == 0:
        raise ValueError(f"image of {x.shape[1]} x {x.shape[2]} pixels is smaller than one {unit} x {unit} neighbourhood")
    x = x[:, :Hh, :Ww]
    x = (x - torch.tensor(mean).view(3, 1, 1)) / torch.tensor(std).view(3, 1, 1)
    h, w = Hh // patch, Ww // patch
    # [3, h/m, m, p, w/m, m, p] -> [h/m, w/m, m, m, 3, p, p]
    x = x.view(3, h // merge, merge, patch, w // merge, merge, patch).permute(1, 4, 2, 5, 0, 3, 6)
    return x.reshape(h * w, 3 * patch * patch).contiguous(), torch.tensor([[1, h, w]], dtype=torch.int64)


def image_rows(ids: torch.Tensor, image_token_id: int) -> torch.Tensor:
    """Rows of a packed id vector that hold image placeholder tokens."""
    return (ids == image_token_id).nonzero(as_tuple=True)[0]
