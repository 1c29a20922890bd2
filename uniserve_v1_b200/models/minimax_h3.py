"""MiniMax-H3 / FastH3-shaped video + audio diffusion transformer.

Packed sequence, dense compute layout ``[video | audio | text | conditions |
padding]`` (generated rows first so sequence-parallel intervals do not move with
the prompt length; unit 64 rows).  Every row carries rotary coordinates (time,
height, width), a tag (video 0, text 1, audio 2) and a timestep group (video 0,
audio 1, visual condition 2, audio condition 3); its AdaLN modulation row is
``3 * group + tag``.

Block::

    n  = rmsnorm(h) * (1 + scale_a[row]) + shift_a[row]
    u  = to_out(attn(qk_norm_rope(to_q(n), to_k(n)), to_v(n)))   # 96 of 128 channels rotated
    r  = h + gate_a[row] * u ;  n2 = rmsnorm(r) * (1 + scale_m[row]) + shift_m[row]
    h  = r + gate_m[row] * ff2(value * silu(gate))               # value rows first, stepwise rounding

Sequence parallelism (Ulysses): rows are split into contiguous intervals; around
attention rows are traded for heads.  Exchange projection: every rank projects
its own rows for all heads (the fused QKV weight is ordered by destination rank)
and the head blocks travel; the attention output travels back before ``to_out``.
The baseline path uses ``all_to_all``; with a peer heap attached the projection
GEMM scatters its tiles into the owners' buffers from its epilogue and ``to_out``
pulls its activation tiles from the peers with TMA (see parallel/ulysses.py).

Reference behaviour: crates/models/src/minimax_h3/transformer.rs:260-352, :909-1013,
packing.rs:1-78, modulation.rs:1-49, crates/nn/src/modules/adaln.rs:1-26,
crates/nn/src/modules/ulysses.rs:1-27 (reference project paths).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..ops import functional as F
from ..ops import reference as R
from ..ops.attention import varlen_attention
from ..parallel.context import ParallelContext

TAG_VIDEO, TAG_TEXT, TAG_AUDIO = 0, 1, 2
GROUP_VIDEO, GROUP_AUDIO, GROUP_VCOND, GROUP_ACOND = 0, 1, 2, 3
SLOT_SHIFT_A, SLOT_SCALE_A, SLOT_GATE_A, SLOT_SHIFT_M, SLOT_SCALE_M, SLOT_GATE_M = range(6)


@dataclass
class H3Config:
    hidden_size: int = 5376
    num_heads: int = 56
    head_dim: int = 128
    num_layers: int = 50
    ffn_size: int = 14336
    text_dim: int = 5120
    refiner_layers: int = 2
    refiner_heads: int = 56
    latent_channels: int = 24
    audio_channels: int = 32
    rope_freqs_per_axis: int = 16
    rope_theta: float = 10000.0
    time_embed_dim: int = 2688
    sinusoid_dim: int = 256
    eps: float = 1e-6
    # VAE geometry (reference: 16x spatial, 4x temporal, clips of 17 frames -> 5 latent frames)
    vae_spatial: int = 16
    vae_temporal_frames: int = 17
    vae_latent_frames: int = 5
    audio_latents_per_second: int = 40
    fps: int = 24
    cond_level_visual: float = 0.999
    cond_level_audio: float = 1.0
    # Video sparse attention (sparse students): fraction of the video key tiles a query
    # tile does NOT read; 0 = dense attention.  Tiles are 128 rows.
    vsa_sparsity: float = 0.0
    # Feed-forward projections in FP8 (E4M3): per-tensor weight scale, per-row dynamic
    # activation scale (the reference's "FP8 MLPs" deployment); attention stays bf16.
    mlp_fp8: bool = False

    @property
    def patch_width(self) -> int:
        return self.latent_channels * 4

    @classmethod
    def tiny(cls) -> "H3Config":
        return cls(hidden_size=256, num_heads=2, head_dim=128, num_layers=2, ffn_size=512,
                   text_dim=128, refiner_layers=1, refiner_heads=2, latent_channels=4,
                   audio_channels=8, time_embed_dim=128, sinusoid_dim=64)

    def latent_shape(self, frames: int, width: int, height: int):
        """Latent grid of a clip.  Frame counts follow the rule 17n + 5; each clip
        of 17 frames gives 5 latent frames and the 5-frame tail 2 more
        (124 frames -> 37 latent frames; 1344x768 -> 84x48 latent, 1008 tokens each)."""
        n = max(0, (frames - 5)) // self.vae_temporal_frames
        lf = self.vae_latent_frames * n + 2
        return lf, height // self.vae_spatial, width // self.vae_spatial

    def audio_rows(self, frames: int) -> int:
        """Audio latent rows of a clip: 40 latents per second, two channels."""
        import math
        return 2 * int(math.ceil(frames / self.fps * self.audio_latents_per_second))


# ------------------------------------------------------------------ schedules --
def shift_sigma(u: float, shift: float) -> float:
    return shift * u / (1.0 + (shift - 1.0) * u)


def dmd_ladder(rungs=(999, 874, 749, 624, 500, 375, 250, 125), shift: float = 10.0):
    """FastH3 distilled ladder: rungs/1000 shifted in FP64, plus the endpoint 0."""
    return [shift_sigma(r / 1000.0, shift) for r in rungs] + [0.0]


def uniform_schedule(steps: int = 50, shift: float = 12.0):
    """Base schedule: uniform grid shifted in FP32, duplicates removed."""
    out = []
    for i in range(steps):
        s = float(torch.tensor(shift_sigma(1.0 - i / steps, shift), dtype=torch.float32))
        if not out or s != out[-1]:
            out.append(s)
    return out + [0.0]


def sinusoidal(t: torch.Tensor, dim: int) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32,
                                                        device=t.device) / half)
    ang = t.float()[:, None] * 1000.0 * freqs[None]
    return torch.cat([ang.cos(), ang.sin()], -1)


# -------------------------------------------------------------------- packing --
@dataclass
class H3Layout:
    """Row bookkeeping of one request in the dense compute layout."""
    n_video: int
    n_audio: int
    n_text: int
    n_cond: int
    rows: int                 # padded total (multiple of 64 * sp)
    used: int                 # rows attention may use as keys
    latent: tuple             # (frames, h, w) of the video latent grid
    coords: torch.Tensor      # [3, rows] fp32
    mod_index: torch.Tensor   # [rows] int32 = 3 * group + tag
    sp: int = 1
    tile_sizes: Optional[torch.Tensor] = None      # VSA: valid rows of each 128-row tile
    tile_segments: Optional[torch.Tensor] = None   # VSA: 0 = video tile, -1 = read by every query
    tile_keep: Optional[torch.Tensor] = None       # VSA: tiles kept per segment

    @property
    def rows_own(self) -> int:
        return self.rows // self.sp

    def interval(self, rank: int):
        return rank * self.rows_own, (rank + 1) * self.rows_own

    def rope_table(self, inv_freq):
        """(cos, sin) table of the rows' rotary factors, built once per layout (CUDA only)."""
        t = getattr(self, "_rope_table", None)
        if t is None and self.coords.is_cuda:
            t = self._rope_table = F.rope3_table(self.coords, inv_freq)
        return t

    def cu(self, device):
        """Cumulative lengths of the one packed sequence: (queries = all rows,
        keys = the rows in use); built once per layout."""
        c = getattr(self, "_cu", None)
        if c is None or c[0].device != torch.device(device):
            c = (torch.tensor([0, self.rows], dtype=torch.int32, device=device),
                 torch.tensor([0, self.used], dtype=torch.int32, device=device))
            self._cu = c
        return c


def build_layout(cfg: H3Config, latent_frames: int, lat_h: int, lat_w: int, n_audio: int,
                 n_text: int, sp: int = 1, n_cond: int = 0, device="cpu") -> H3Layout:
    hp, wp = lat_h // 2, lat_w // 2
    n_video = latent_frames * hp * wp
    used = n_video + n_audio + n_text + n_cond
    vsa = cfg.vsa_sparsity > 0
    unit = (128 if vsa else 64) * sp
    rows = (used + unit - 1) // unit * unit
    coords = torch.zeros(3, rows, dtype=torch.float32)
    f = torch.arange(latent_frames, dtype=torch.float32)
    y = torch.arange(hp, dtype=torch.float32)
    x = torch.arange(wp, dtype=torch.float32)
    grid = torch.stack(torch.meshgrid(f, y, x, indexing="ij"), 0).reshape(3, -1)
    coords[:, :n_video] = grid
    # audio rows advance along time only, at the latent-frame rate rescaled 5/3
    if n_audio:
        coords[0, n_video:n_video + n_audio] = torch.arange(n_audio, dtype=torch.float32) * \
            (latent_frames / max(n_audio, 1))
    tags = torch.full((rows,), TAG_TEXT, dtype=torch.int32)
    groups = torch.zeros(rows, dtype=torch.int32)
    tags[:n_video] = TAG_VIDEO
    tags[n_video:n_video + n_audio] = TAG_AUDIO
    groups[n_video:n_video + n_audio] = GROUP_AUDIO
    c0 = n_video + n_audio + n_text
    tags[c0:c0 + n_cond] = TAG_VIDEO
    groups[c0:c0 + n_cond] = GROUP_VCOND
    mod = 3 * groups + tags
    lay = H3Layout(n_video, n_audio, n_text, n_cond, rows, used, (latent_frames, lat_h, lat_w),
                   coords.to(device), mod.to(device), sp)
    if vsa:
        tiles = rows // 128
        t0 = torch.arange(tiles, dtype=torch.int32) * 128
        sizes = (used - t0).clamp(0, 128).to(torch.int32)
        seg = torch.where(t0 + 128 <= n_video, 0, -1).to(torch.int32)
        n_vid_tiles = int((seg == 0).sum())
        keep = torch.zeros(tiles, dtype=torch.int32)
        keep[0] = max(1, math.ceil((1.0 - cfg.vsa_sparsity) * n_vid_tiles))
        lay.tile_sizes, lay.tile_segments, lay.tile_keep = (sizes.to(device), seg.to(device),
                                                            keep.to(device))
    return lay


# -------------------------------------------------------------------- weights --
@dataclass
class H3Block:
    qkv: torch.Tensor        # [3 * hidden, hidden], rows grouped by destination rank
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    to_out: torch.Tensor     # [hidden, heads * head_dim]
    ff1: torch.Tensor        # [2 * ffn, hidden] value rows, then gate rows
    ff2: torch.Tensor        # [hidden, ffn]
    # With sparse attention ``qkv`` carries a fourth projection per rank
    # (to_gate_compress): rows [q | k | v | gate] per destination rank.
    ff1_scale: Optional[float] = None   # set: ff1 / ff2 hold E4M3 bytes with these scales
    ff2_scale: Optional[float] = None


@dataclass
class RefinerBlock:
    norm1: torch.Tensor
    qkv: torch.Tensor
    to_out: torch.Tensor
    norm2: torch.Tensor
    ff1: torch.Tensor
    ff2: torch.Tensor


class H3Transformer:
    def __init__(self, cfg: H3Config, device="cpu", dtype=torch.bfloat16,
                 ctx: Optional[ParallelContext] = None):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.ctx = ctx or ParallelContext.single()
        # Rows are split over the sequence ranks: "ulysses" (heads travel around attention),
        # "gather" (queries stay, K and V rows are all-gathered, every head is local) or
        # both ("sequence": Ulysses inside each gather place - the place's rows meet on
        # every member for its share of the heads, and K / V of that share are gathered
        # across the places; family.rs:607-690, reference project path).
        uly, gat = self.ctx.axis("ulysses").size, self.ctx.axis("gather").size
        self.seq_axis = "sequence" if (uly > 1 and gat > 1) else ("gather" if gat > 1
                                                                   else "ulysses")
        if self.seq_axis == "sequence":
            self.sp = uly * gat
            self.sp_rank = self.ctx.axis("gather").rank * uly + self.ctx.axis("ulysses").rank
        else:
            self.sp = self.ctx.axis(self.seq_axis).size
            self.sp_rank = self.ctx.axis(self.seq_axis).rank
        self.head_split = uly
        self.gather_places = gat
        assert cfg.num_heads % self.head_split == 0, "heads must divide over the Ulysses group"
        self.heads_local = cfg.num_heads // self.head_split
        # Layer split: contiguous shares of the blocks along the "layer" axis; a stage
        # hands its rows to the next by point-to-point messages and the last stage
        # broadcasts the velocity rows (transformer.rs:934-953, reference project path).
        lay = self.ctx.axis("layer")
        self.pp, self.pp_rank, self.pp_axis = lay.size, lay.rank, lay
        per = (cfg.num_layers + self.pp - 1) // self.pp
        self.block_lo = min(cfg.num_layers, self.pp_rank * per)
        self.block_hi = min(cfg.num_layers, (self.pp_rank + 1) * per)
        self.inv_freq = R.rope_inv_freq(2 * cfg.rope_freqs_per_axis, cfg.rope_theta, self.device)
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        self.blocks: list = []
        self.refiner: list = []
        self.tables: list = []        # per level: [layers] of [12 * 6, hidden] fp32
        self.tables_out: list = []    # per level: [12 * 2, hidden] fp32
        self.ulysses = None           # parallel.ulysses.FusedUlysses when a peer heap is attached
        self.probe = None             # engine.profiling.ProbeRing: per-phase fence probes

    # --------------------------------------------------------------- weights --
    def init_random(self, seed: int = 0, std: float = 0.02) -> "H3Transformer":
        cfg, dev, dt = self.cfg, self.device, self.dtype
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        H, D, Fn = cfg.hidden_size, cfg.head_dim, cfg.ffn_size

        def rnd(*shape, dtype=dt, s=std):
            return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * s).to(dtype)

        ones = lambda n: torch.ones(n, device=dev, dtype=dt)
        self.proj_in = rnd(H, cfg.patch_width, dtype=torch.float32)
        self.audio_proj_in = rnd(H, cfg.audio_channels, dtype=torch.float32)
        self.context_embedder = rnd(H, cfg.text_dim)
        for _ in range(cfg.refiner_layers):
            self.refiner.append(RefinerBlock(ones(H), rnd(3 * H, H), rnd(H, H), ones(H),
                                             rnd(2 * Fn, H), rnd(H, Fn)))
        self.refiner_norm = ones(H)
        for _ in range(cfg.num_layers):
            inner = cfg.num_heads * D     # 56 x 128 = 7168 on a 5376-wide stream
            q, k, v = rnd(inner, H), rnd(inner, H), rnd(inner, H)
            gate = rnd(inner, H) if cfg.vsa_sparsity > 0 else None
            blk = H3Block(self._group_qkv(q, k, v, gate), ones(D), ones(D), rnd(H, inner),
                          rnd(2 * Fn, H), rnd(H, Fn))
            own = self.block_lo <= len(self.blocks) < self.block_hi
            if own and cfg.mlp_fp8:
                from ..ops.fp8 import quantize_weight_tensor
                blk.ff1, blk.ff1_scale = quantize_weight_tensor(blk.ff1)
                blk.ff2, blk.ff2_scale = quantize_weight_tensor(blk.ff2)
            self.blocks.append(blk if own else None)
        self.proj_out = rnd(cfg.patch_width, H, dtype=torch.float32)
        self.audio_proj_out = rnd(cfg.audio_channels, H, dtype=torch.float32)
        # time embedder + per-block AdaLN projections (FP32); used to build level tables
        self.time_w1 = rnd(cfg.time_embed_dim, cfg.sinusoid_dim, dtype=torch.float32)
        self.time_w2 = rnd(cfg.time_embed_dim, cfg.time_embed_dim, dtype=torch.float32)
        self._adaln_seed = seed + 1
        return self

    def _group_qkv(self, q, k, v, gate=None):
        """Row order [rank 0: q heads, k heads, v heads (, gate heads) | rank 1: ... ] so
        the projection output is already blocked by destination rank."""
        P, hl, D = self.head_split, self.heads_local, self.cfg.head_dim
        parts = []
        for p in range(P):
            sl = slice(p * hl * D, (p + 1) * hl * D)
            parts += [q[sl], k[sl], v[sl]] + ([gate[sl]] if gate is not None else [])
        return torch.cat(parts, 0).contiguous()

    def build_level_tables(self, video_sigmas, audio_sigmas) -> None:
        """Precomputes, per schedule level, each block's modulation table
        [12 rows (3 * group + tag) x 6 vectors, hidden] and the output table.
        AdaLN projection weights are generated per block and dropped: only the
        tables stay resident (reference: TimestepTable, modulation.rs:1-30)."""
        cfg, dev = self.cfg, self.device
        H, Te = cfg.hidden_size, cfg.time_embed_dim
        g = torch.Generator(device=dev)
        g.manual_seed(self._adaln_seed)
        levels = len(video_sigmas)
        t = torch.tensor([[1.0 - video_sigmas[i], 1.0 - audio_sigmas[i],
                           1.0 - cfg.cond_level_visual, 1.0 - cfg.cond_level_audio]
                          for i in range(levels)], dtype=torch.float32, device=dev)   # [L, 4]
        emb = sinusoidal(t.reshape(-1), cfg.sinusoid_dim)
        temb = torch.nn.functional.silu(emb @ self.time_w1.t()) @ self.time_w2.t()     # [L*4, Te]
        act = torch.nn.functional.silu(temb)
        self.tables = [[] for _ in range(levels)]
        for _ in range(cfg.num_layers):
            w = torch.randn(18 * H, Te, generator=g, device=dev, dtype=torch.float32) * 0.02
            mod = (act @ w.t()).view(levels, 4, 3, 6, H)          # [L, group, tag, 6, H]
            for lv in range(levels):
                self.tables[lv].append(mod[lv].reshape(12 * 6, H).contiguous())
            del w
        w = torch.randn(6 * H, Te, generator=g, device=dev, dtype=torch.float32) * 0.02
        mo = (act @ w.t()).view(levels, 4, 3, 2, H)
        self.tables_out = [mo[lv].reshape(12 * 2, H).contiguous() for lv in range(levels)]

    # ---------------------------------------------------------------- refiner --
    def refine_text(self, text_features: torch.Tensor) -> torch.Tensor:
        """context_embedder then pre-norm blocks with dense bidirectional attention
        and SwiGLU, then a final norm; not sequence-split (refiner.rs:1-26)."""
        cfg = self.cfg
        x = F.linear(text_features.to(self.dtype), self.context_embedder)
        n = x.shape[0]
        Hh, D = cfg.refiner_heads, cfg.hidden_size // cfg.refiner_heads
        cu = torch.tensor([0, n], dtype=torch.int32, device=x.device)
        for b in self.refiner:
            h = F.rmsnorm(x, b.norm1, cfg.eps)
            qkv = F.linear(h, b.qkv).view(n, 3 * Hh, D)
            a = self._dense_attention(qkv[:, :Hh], qkv[:, Hh:2 * Hh], qkv[:, 2 * Hh:], cu, cu, n, n)
            x = x + F.linear(a.reshape(n, Hh * D), b.to_out)
            h = F.rmsnorm(x, b.norm2, cfg.eps)
            x = x + F.linear(F.linear_gated(h, b.ff1), b.ff2)
        return F.rmsnorm(x, self.refiner_norm, cfg.eps)

    def _dense_attention(self, q, k, v, cu_q, cu_k, max_q, max_k):
        D = q.shape[-1]
        if q.is_cuda and D != 128:
            return R.varlen_attention(q, k, v, cu_q, cu_k, 1.0 / math.sqrt(D), False)
        return varlen_attention(q, k, v, cu_q, cu_k, max_q, max_k, 1.0 / math.sqrt(D), False)

    # ------------------------------------------------------------------ inputs --
    def embed_rows(self, layout: H3Layout, video_latent, audio_latent, text_rows,
                   cond_rows=None) -> torch.Tensor:
        """Own interval of the packed rows [rows_own, hidden] in bf16 (FP32 input
        projections, narrowed once)."""
        from ..ops.diffusion import patchify
        cfg = self.cfg
        lo, hi = layout.interval(self.sp_rank)
        parts = []
        v = patchify(video_latent.float()) @ self.proj_in.t()
        a = audio_latent.float() @ self.audio_proj_in.t()
        parts = [v, a, text_rows.float()]
        if cond_rows is not None:
            parts.append(cond_rows.float())
        x = torch.cat(parts, 0)
        pad = layout.rows - x.shape[0]
        if pad:
            x = torch.cat([x, torch.zeros(pad, cfg.hidden_size, device=x.device)], 0)
        return x[lo:hi].to(self.dtype).contiguous()

    # ----------------------------------------------------------------- forward --
    def _range(self, name: str, tag: int = 0):
        """Fence-probe range around a phase of a block (no-op without a probe ring)."""
        import contextlib
        if self.probe is None:
            return contextlib.nullcontext()
        probe = self.probe

        @contextlib.contextmanager
        def rng():
            probe.mark(name + ".begin", tag)
            try:
                yield
            finally:
                probe.mark(name + ".end", tag)
        return rng()

    def _attention(self, blk: H3Block, n: torch.Tensor, layout: H3Layout) -> torch.Tensor:
        cfg = self.cfg
        if self.seq_axis == "gather" and self.sp > 1:
            return self._attention_gather(blk, n, layout)
        hl, D, P = self.heads_local, cfg.head_dim, self.head_split
        hybrid = self.seq_axis == "sequence"
        vsa = cfg.vsa_sparsity > 0
        assert not (hybrid and vsa), "block-sparse attention runs on one sequence axis"
        if hybrid:
            P_, ro_ = P, n.shape[0]
            coords = layout.coords[:, self.ctx.axis("gather").rank * P_ * ro_:
                                   (self.ctx.axis("gather").rank + 1) * P_ * ro_].contiguous()
        W = (4 if vsa else 3) * hl * D
        if P > 1 and self.ulysses is not None and n.is_cuda and not vsa and not hybrid:
            return self.ulysses.attention(self, blk, n, layout)
        qkv = F.linear(n, blk.qkv)                               # [rows_own, P * W]
        if P > 1:
            ro = qkv.shape[0]
            send = qkv.view(ro, P, W).permute(1, 0, 2).contiguous()
            full = self.ctx.all_to_all(send, "ulysses").view(P * ro, W)
        else:
            full = qkv
        rows = full.shape[0]
        q, k, v = full[:, :hl * D], full[:, hl * D:2 * hl * D], full[:, 2 * hl * D:]
        if hybrid:
            # rows of this gather place, this member's heads; keys and values of the
            # other places arrive by all-gather over the gather axis
            F.qk_norm_rope3_(q, k, blk.q_norm, blk.k_norm, coords, self.inv_freq, hl, hl, D,
                             cfg.rope_freqs_per_axis, cfg.eps)
            k_all = self.ctx.all_gather_rows(k.contiguous(), "gather")
            v_all = self.ctx.all_gather_rows(v.contiguous(), "gather")
            dev = n.device
            cu_q = torch.tensor([0, rows], dtype=torch.int32, device=dev)
            cu_k = torch.tensor([0, layout.used], dtype=torch.int32, device=dev)
            att = self._dense_attention(q.reshape(rows, hl, D), k_all.view(-1, hl, D),
                                        v_all.view(-1, hl, D), cu_q, cu_k, rows,
                                        layout.used).reshape(rows, hl * D)
        else:
            F.qk_norm_rope3_(q, k, blk.q_norm, blk.k_norm, layout.coords, self.inv_freq, hl, hl,
                             D, cfg.rope_freqs_per_axis, cfg.eps,
                             table=layout.rope_table(self.inv_freq))
        if hybrid:
            pass
        elif vsa:
            from ..ops import vsa as V
            v3 = full[:, 2 * hl * D:3 * hl * D].view(rows, hl, D)
            g3 = full[:, 3 * hl * D:].view(rows, hl, D)
            att = V.vsa_attention(q.view(rows, hl, D), k.view(rows, hl, D), v3, g3,
                                  layout.tile_sizes, layout.tile_segments, layout.tile_keep,
                                  self.scale).reshape(rows, hl * D)
        else:
            cu_q, cu_k = layout.cu(n.device)
            att = self._dense_attention(q.view(rows, hl, D), k.view(rows, hl, D),
                                        v.view(rows, hl, D), cu_q, cu_k, rows,
                                        layout.used).reshape(rows, hl * D)
        if P > 1:
            ro = rows // P
            back = self.ctx.all_to_all(att.view(P, ro, hl * D), "ulysses")   # [P(heads), ro, hl*D]
            att = back.permute(1, 0, 2).reshape(ro, P * hl * D).contiguous()
        return F.linear(att, blk.to_out)

    def _attention_gather(self, blk: H3Block, n: torch.Tensor, layout: H3Layout) -> torch.Tensor:
        """All-gather sequence parallelism: this rank's rows are the queries; K and V of
        every interval are all-gathered along the gather axis; all heads are local
        (crates/models/src/minimax_h3/transformer.rs:299-314, reference project path)."""
        cfg = self.cfg
        H_, D = cfg.num_heads, cfg.head_dim
        ro = n.shape[0]
        lo, hi = layout.interval(self.sp_rank)
        qkv = F.linear(n, blk.qkv)                               # [rows_own, 3 * heads * D]
        q, k, v = qkv[:, :H_ * D], qkv[:, H_ * D:2 * H_ * D], qkv[:, 2 * H_ * D:]
        coords = layout.coords[:, lo:hi].contiguous()
        F.qk_norm_rope3_(q, k, blk.q_norm, blk.k_norm, coords, self.inv_freq, H_, H_, D,
                         cfg.rope_freqs_per_axis, cfg.eps)
        k_all = self.ctx.all_gather_rows(k.contiguous(), "gather")
        v_all = self.ctx.all_gather_rows(v.contiguous(), "gather")
        dev = n.device
        cu_q = torch.tensor([0, ro], dtype=torch.int32, device=dev)
        cu_k = torch.tensor([0, layout.used], dtype=torch.int32, device=dev)
        att = self._dense_attention(q.reshape(ro, H_, D), k_all.view(-1, H_, D),
                                    v_all.view(-1, H_, D), cu_q, cu_k, ro, layout.used)
        return F.linear(att.reshape(ro, H_ * D), blk.to_out)

    def forward(self, h: torch.Tensor, layout: H3Layout, level: int):
        """h: own rows [rows_own, hidden] bf16.  Returns FP32 velocity rows of the
        own interval: (video part [*, patch_width], audio part [*, audio_channels])
        with the row ranges they cover."""
        cfg = self.cfg
        lo, hi = layout.interval(self.sp_rank)
        idx = layout.mod_index[lo:hi].contiguous()
        if self.pp > 1 and self.pp_rank > 0:
            h = self._stage_recv(h)
        for b in range(self.block_lo, self.block_hi):
            blk = self.blocks[b]
            table = self.tables[level][b]
            with self._range("norm_a", b):
                n = F.modulated_rmsnorm(h, None, table, idx, 6, SLOT_SHIFT_A, SLOT_SCALE_A,
                                        cfg.eps)
            with self._range("attention", b):
                u = self._attention(blk, n, layout)
            with self._range("gate_norm_m", b):
                F.gated_residual_(h, u, table, idx, 6, SLOT_GATE_A)
                n2 = F.modulated_rmsnorm(h, None, table, idx, 6, SLOT_SHIFT_M, SLOT_SCALE_M,
                                         cfg.eps)
            if blk.ff1_scale is not None:
                from ..ops.fp8 import linear_fp8
                with self._range("ff1", b):
                    hid = linear_fp8(n2, blk.ff1, blk.ff1_scale, gated=True, stepwise=True)
                with self._range("ff2", b):
                    ff = linear_fp8(hid, blk.ff2, blk.ff2_scale)
            else:
                with self._range("ff1", b):
                    hid = F.linear_gated(n2, blk.ff1, stepwise=True)
                with self._range("ff2", b):
                    ff = F.linear(hid, blk.ff2)
            with self._range("gate_m", b):
                F.gated_residual_(h, ff, table, idx, 6, SLOT_GATE_M)
        v_lo, v_hi = max(lo, 0), min(hi, layout.n_video)
        a_lo, a_hi = max(lo, layout.n_video), min(hi, layout.n_video + layout.n_audio)
        nv, na = max(v_hi, v_lo) - v_lo, max(a_hi, a_lo) - a_lo
        last = self.pp - 1
        if self.pp > 1 and self.pp_rank != last:
            self._stage_send(h)
            vel_v = torch.empty(nv, cfg.patch_width, dtype=torch.float32, device=h.device)
            vel_a = torch.empty(na, cfg.audio_channels, dtype=torch.float32, device=h.device)
        else:
            out = F.modulated_rmsnorm(h, None, self.tables_out[level], idx, 2, 0, 1,
                                      cfg.eps).float()
            vel_v = out[v_lo - lo:v_lo - lo + nv] @ self.proj_out.t()
            vel_a = out[a_lo - lo:a_lo - lo + na] @ self.audio_proj_out.t()
        if self.pp > 1:      # every stage advances the same latents
            vel_v = self.ctx.broadcast(vel_v.contiguous(), last, "layer")
            vel_a = self.ctx.broadcast(vel_a.contiguous(), last, "layer")
        return vel_v, vel_a

    def _stage_send(self, h: torch.Tensor) -> None:
        import torch.distributed as dist
        dist.send(h.contiguous(), self.pp_axis.ranks[self.pp_rank + 1], group=self.pp_axis.group)

    def _stage_recv(self, like: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        h = torch.empty_like(like)
        dist.recv(h, self.pp_axis.ranks[self.pp_rank - 1], group=self.pp_axis.group)
        return h

    def clone_to(self, device, dtype) -> "H3Transformer":
        """The same weights on another device / in another dtype (tests compare a
        bf16 GPU model with its FP32 CPU twin)."""
        import copy
        import dataclasses
        o = H3Transformer(self.cfg, device, dtype, self.ctx)
        def mv(t, keep=False):
            if not isinstance(t, torch.Tensor):
                return t                                    # scales, absent tensors
            if t.dtype == torch.uint8:
                keep = True                                 # quantised bytes stay bytes
            return t.to(device=o.device, dtype=t.dtype if keep else dtype)
        for name in ("proj_in", "audio_proj_in", "proj_out", "audio_proj_out", "time_w1", "time_w2"):
            setattr(o, name, mv(getattr(self, name), True))
        o.context_embedder = mv(self.context_embedder)
        o.refiner_norm = mv(self.refiner_norm)
        o.refiner = [RefinerBlock(*[mv(getattr(b, f.name)) for f in dataclasses.fields(b)])
                     for b in self.refiner]
        o.blocks = [None if b is None else
                    H3Block(*[mv(getattr(b, f.name)) for f in dataclasses.fields(b)])
                    for b in self.blocks]
        o._adaln_seed = self._adaln_seed
        o.tables = [[t.to(o.device) for t in lv] for lv in self.tables]
        o.tables_out = [t.to(o.device) for t in self.tables_out]
        return o

    def weight_bytes(self) -> int:
        n = 0
        for b in self.blocks:
            if b is not None:
                n += b.qkv.numel() + b.to_out.numel() + b.ff1.numel() + b.ff2.numel()
        return n * 2


# ------------------------------------------------------------------- denoiser --
@dataclass
class DenoiseState:
    layout: H3Layout
    video: torch.Tensor     # [C, F, H, W] fp32 latents (identical on every rank)
    audio: torch.Tensor     # [n_audio, audio_channels] fp32
    text_rows: torch.Tensor
    step: int = 0
    seed: int = 0
    cond_rows: Optional[torch.Tensor] = None    # [n_cond, hidden] FP32, fixed over the steps


class Denoiser:
    """Runs the sampler: every step is one transformer evaluation on every rank
    of the sequence group, the velocity rows are all-gathered in sequence order
    and each rank advances the same FP32 latents (denoiser.rs:36-43, :786-805)."""

    def __init__(self, model: H3Transformer, video_sigmas=None, audio_sigmas=None):
        self.model = model
        self.video_sigmas = video_sigmas or dmd_ladder(shift=10.0)
        self.audio_sigmas = audio_sigmas or dmd_ladder(shift=3.0)
        assert len(self.video_sigmas) == len(self.audio_sigmas)
        self.steps = len(self.video_sigmas) - 1
        if len(model.tables) != self.steps:
            model.build_level_tables(self.video_sigmas[:-1], self.audio_sigmas[:-1])

    def prepare(self, seed: int, latent_frames: int, lat_h: int, lat_w: int, n_audio: int,
                text_features: torch.Tensor, conditions=None) -> DenoiseState:
        """``conditions``: (latent frame index, latent [C, 1, lat_h, lat_w]) pairs.  A keyframe
        names the frame it pins (0, or -1 for the last) and sits at that frame's rotary
        coordinates; a reference image has index ``None`` and sits on the same spatial grid one
        time unit apart from the others, before the clip (the k-th of n at time k - n); a
        reference clip is the same with several latent frames, spread over its unit.  A
        reference track is (None, latent rows [n, audio channels]): audio rows of the clean
        audio-condition group spread over its time unit.  The rows follow the text rows, the
        visual ones in the visual-condition timestep group, and stay as encoded through every
        step."""
        from ..ops.diffusion import patchify, philox_normal
        m, cfg = self.model, self.model.cfg
        dev = m.device
        conditions = list(conditions or [])
        per = (lat_h // 2) * (lat_w // 2)
        sizes = [lat.shape[0] if lat.dim() == 2 else per * (lat.shape[1] if lat.dim() == 4 else 1)
                 for _, lat in conditions]
        layout = build_layout(cfg, latent_frames, lat_h, lat_w, n_audio, text_features.shape[0],
                              m.sp, sum(sizes), dev)
        cond_rows = None
        if conditions:
            refs = [j for j, (f, _) in enumerate(conditions) if f is None]
            at = layout.n_video + layout.n_audio + layout.n_text
            rows = []
            for k, (frame, latent) in enumerate(conditions):
                own = layout.coords[:, at:at + sizes[k]]
                clock = float(refs.index(k) - len(refs)) if frame is None else None
                if latent.dim() == 2:
                    # a reference track: audio rows, clean, along time from its place before
                    # the clip at the generated audio's rate
                    if frame is not None or latent.shape[1] != cfg.audio_channels:
                        raise ValueError(f"a reference track is [rows, {cfg.audio_channels}] "
                                         "without a frame to pin")
                    own.zero_()
                    own[0] = clock + torch.arange(sizes[k], device=dev, dtype=torch.float32) / \
                        max(sizes[k], 1)
                    layout.mod_index[at:at + sizes[k]] = 3 * GROUP_ACOND + TAG_AUDIO
                    rows.append(latent.to(dev).float() @ m.audio_proj_in.t())
                else:
                    fr = latent.shape[1] if latent.dim() == 4 else 0
                    if tuple(latent.shape) != (cfg.latent_channels, fr, lat_h, lat_w) or \
                            fr < 1 or (frame is not None and fr != 1):
                        raise ValueError(f"a keyframe latent is [{cfg.latent_channels}, 1, "
                                         f"{lat_h}, {lat_w}] (a reference clip has more "
                                         f"frames), got {tuple(latent.shape)}")
                    if frame is None:
                        # a reference clip's latent frames share its time unit
                        own.copy_(layout.coords[:, :per].repeat(1, fr))
                        own[0] = clock + torch.arange(fr, device=dev, dtype=torch.float32
                                                      ).repeat_interleave(per) / fr
                    else:
                        frame = frame % latent_frames
                        own.copy_(layout.coords[:, frame * per:(frame + 1) * per])
                    rows.append(patchify(latent.to(dev).float()) @ m.proj_in.t())
                at += sizes[k]
            cond_rows = torch.cat(rows, 0)
        video = philox_normal((cfg.latent_channels, latent_frames, lat_h, lat_w), seed, 0, 1.0, dev)
        audio = philox_normal((n_audio, cfg.audio_channels), seed, 1, 1.0, dev)
        text_rows = m.refine_text(text_features.to(dev))
        return DenoiseState(layout, video, audio, text_rows, 0, seed, cond_rows)

    def step(self, st: DenoiseState) -> DenoiseState:
        from ..ops.diffusion import scaled_add_, unpatchify
        m, cfg, i = self.model, self.model.cfg, st.step
        h = m.embed_rows(st.layout, st.video, st.audio, st.text_rows, st.cond_rows)
        vel_v, vel_a = m.forward(h, st.layout, i)
        if m.sp > 1:
            vel_v, vel_a = self._gather(vel_v, vel_a, st.layout)
        Fr, H, W = st.layout.latent
        v_lat = unpatchify(vel_v.contiguous(), cfg.latent_channels, Fr, H, W)
        scaled_add_(st.video, v_lat, self.video_sigmas[i + 1] - self.video_sigmas[i])
        scaled_add_(st.audio, vel_a.contiguous(), self.audio_sigmas[i + 1] - self.audio_sigmas[i])
        st.step += 1
        return st

    def _gather(self, vel_v, vel_a, layout: H3Layout):
        """All-gather of the velocity rows in sequence order (ragged: pad to the
        interval length, gather, cut)."""
        m = self.model
        ro = layout.rows_own

        def gather(x, width, total):
            buf = torch.zeros(ro, width, dtype=torch.float32, device=x.device)
            buf[:x.shape[0]] = x
            if m.seq_axis == "sequence":
                allr = m.ctx.all_gather_rows(m.ctx.all_gather_rows(buf, "ulysses"), "gather")
            else:
                allr = m.ctx.all_gather_rows(buf, m.seq_axis)
            allr = allr.view(m.sp, ro, width)
            return allr

        gv = gather(vel_v, m.cfg.patch_width, layout.n_video)
        ga = gather(vel_a, m.cfg.audio_channels, layout.n_audio)
        vs, as_ = [], []
        for r in range(m.sp):
            lo, hi = r * ro, (r + 1) * ro
            nv = max(0, min(hi, layout.n_video) - lo)
            vs.append(gv[r, :nv])
            a_lo, a_hi = max(lo, layout.n_video), min(hi, layout.n_video + layout.n_audio)
            as_.append(ga[r, :max(0, a_hi - a_lo)])
        return torch.cat(vs, 0), torch.cat(as_, 0)

    def run(self, st: DenoiseState) -> DenoiseState:
        while st.step < self.steps:
            self.step(st)
        return st
