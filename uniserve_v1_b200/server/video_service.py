"""Video generation service: the request state machine and the job store.

Phases of a request (crates/engine/src/scheduler/video.rs:1-33, :86-116, reference
project path): ``TextEncode`` -> ``LatentPrepare`` -> ``Denoise`` x steps ->
``VideoDecode`` || ``AudioDecode`` -> ``VideoEncode``, ``AudioEncode`` -> ``Mux``.
A trajectory is resumable at step boundaries: the job keeps (seed, step, latents),
and because the noise is addressable a restarted job redraws identical latents.
Jobs are kept for an hour, within one GiB of results (oldest evicted first).
"""
from __future__ import annotations

import asyncio
import hashlib
import threading
import time
import uuid
from collections import OrderedDict
from typing import Optional

import numpy as np
import torch

from ..models.h3_vae import AudioVaeDecoder, VideoVaeDecoder
from ..models.minimax_h3 import Denoiser, H3Transformer
from ..ops import media as M


class TextEncoder:
    """Prompt -> text features [n, text_dim].  The served family conditions on a
    Qwen3-VL encoder (50 of 64 layers); without its checkpoint the stand-in here
    embeds the prompt's bytes deterministically (hash-seeded normal rows), which
    keeps prompt capacity, caching by key and every downstream shape real."""

    def __init__(self, text_dim: int, max_tokens: int = 512):
        self.text_dim, self.max_tokens = text_dim, max_tokens
        self.cache: OrderedDict = OrderedDict()

    def key(self, prompt: str) -> str:
        return hashlib.sha256(prompt.encode()).hexdigest()

    def encode(self, prompt: str, device) -> torch.Tensor:
        k = self.key(prompt)
        if k in self.cache:
            self.cache.move_to_end(k)
            return self.cache[k].to(device)
        toks = list(prompt.encode())[:self.max_tokens] or [0]
        rows = []
        for i, t in enumerate(toks):
            g = torch.Generator().manual_seed((t << 20) ^ i)
            rows.append(torch.randn(self.text_dim, generator=g))
        feats = torch.stack(rows, 0)
        self.cache[k] = feats
        while len(self.cache) > 64:
            self.cache.popitem(last=False)
        return feats.to(device)


class ModelTextEncoder(TextEncoder):
    """Prompt features from a language model used as an encoder: the residual stream of a
    Qwen3 decoder after ``num_layers`` blocks (the served family reads 50 of 64), one row
    per prompt token.  Same cache and key as the stand-in."""

    def __init__(self, model, tokenizer, num_layers: Optional[int] = None, max_tokens: int = 512):
        super().__init__(model.cfg.hidden_size, max_tokens)
        self.model, self.tokenizer, self.num_layers = model, tokenizer, num_layers

    def encode(self, prompt: str, device) -> torch.Tensor:
        k = self.key(prompt)
        if k in self.cache:
            self.cache.move_to_end(k)
            return self.cache[k].to(device)
        ids = self.tokenizer.encode(prompt)[:self.max_tokens] or [0]
        feats = self.model.encode(ids, self.num_layers).float().cpu()
        self.cache[k] = feats
        while len(self.cache) > 64:
            self.cache.popitem(last=False)
        return feats.to(device)


class VideoJob:
    def __init__(self, prompt: str, plan):
        self.id = "video_" + uuid.uuid4().hex[:24]
        self.prompt, self.plan = prompt, plan
        self.state = "queued"
        self.phase = "Queued"
        self.timings: dict = {}
        self.progress = 0.0
        self.created = int(time.time())
        self.completed_at: Optional[int] = None
        self.error: Optional[str] = None
        self.content: Optional[bytes] = None
        self.step = 0
        self.resumes = 0
        self.resumed_from: Optional[int] = None
        self.cancelled = False
        self._done = threading.Event()
        self._waiters: list = []

    def record(self) -> dict:
        p = self.plan
        return {"id": self.id, "object": "video", "status": self.state, "phase": self.phase,
                "progress": round(self.progress, 3), "created_at": self.created,
                "completed_at": self.completed_at, "size": f"{p.width}x{p.height}",
                "num_frames": p.num_frames, "fps": p.fps, "seconds": f"{p.seconds:.3f}",
                "seed": p.seed, "task": p.task, "error": self.error,
                "bytes": len(self.content) if self.content else None}

    async def wait(self):
        loop = asyncio.get_running_loop()
        await loop.run_in_executor(None, self._done.wait)

    def finish(self, state: str, error: Optional[str] = None):
        self.state, self.error = state, error
        self.completed_at = int(time.time())
        self._done.set()


class VideoService:
    def __init__(self, transformer: H3Transformer, video_vae: VideoVaeDecoder,
                 audio_vae: AudioVaeDecoder, sizes=None, max_seconds: int = 15,
                 retention_s: float = 3600.0, store_bytes: int = 1 << 30, observation=None,
                 video_encoder=None, audio_encoder=None):
        from .video_rules import SIZES
        self.model = transformer
        # keyframe conditions (first / last frame images) are encoded by the VAE's encoder;
        # a deployment without one serves text-to-video only
        self.video_encoder, self.audio_encoder = video_encoder, audio_encoder
        self.tasks = ("t2va", "fl2va", "ref2va") if video_encoder is not None else ("t2va",)
        # Ranks of the sequence group also share the decode work: temporal units
        # are dealt round-robin and the encoded planes gathered on every rank
        # (crates/engine/src/runner/decoder.rs:57-70, reference project path).
        ax = transformer.ctx.axis(getattr(transformer, "seq_axis", "ulysses"))
        self.world, self.rank, self.group = ax.size, ax.rank, ax.group
        self.h2d_bytes = self.d2h_bytes = 0
        self.time_phases = False
        self._copy_stream = None          # device -> host copies of the planes
        self._audio_stream = None         # the audio decoder beside the video decoder
        self._pinned = None               # pinned host buffer of the encoded planes, reused
        self.denoiser = Denoiser(transformer)
        self.steps = self.denoiser.steps
        self.video_vae, self.audio_vae = video_vae, audio_vae
        self.text = TextEncoder(transformer.cfg.text_dim)
        self.sizes = sizes or SIZES
        self.max_seconds = max_seconds
        self.retention_s, self.store_bytes = retention_s, store_bytes
        self.obs = observation
        # Host latent pool: the trajectory of every running job at its last step boundary
        # (step index + video and audio latents, a few tens of MB), so that a job that
        # failed or was interrupted continues from there - on this or on another layout,
        # the latents are whole on every rank (runner/denoiser.rs:62-79, reference path).
        self.latent_pool: OrderedDict = OrderedDict()
        self.latent_pool_bytes = 1 << 30
        self.max_resumes = 2
        self._jobs: OrderedDict = OrderedDict()
        self._queue: list = []
        self._cv = threading.Condition()
        self._stop = False
        self._thread = threading.Thread(target=self._run, name="video-loop", daemon=True)
        self._started = False

    def start(self):
        if not self._started:
            self._started = True
            self._thread.start()

    def stop(self):
        with self._cv:
            self._stop = True
            self._cv.notify_all()

    # ------------------------------------------------------------------- jobs --
    def submit(self, prompt: str, plan) -> VideoJob:
        job = VideoJob(prompt, plan)
        with self._cv:
            self._jobs[job.id] = job
            self._queue.append(job)
            self._cv.notify_all()
        self.start()
        return job

    def get(self, job_id: str) -> Optional[VideoJob]:
        self._evict()
        return self._jobs.get(job_id)

    def jobs(self) -> list:
        self._evict()
        return list(self._jobs.values())

    def delete(self, job_id: str) -> bool:
        with self._cv:
            job = self._jobs.pop(job_id, None)
            if job is None:
                return False
            job.cancelled = True
            if job in self._queue:
                self._queue.remove(job)
                job.finish("failed", "cancelled")
        return True

    def _evict(self):
        now = time.time()
        with self._cv:
            for jid, j in list(self._jobs.items()):
                if j.completed_at and now - j.completed_at > self.retention_s:
                    del self._jobs[jid]
            total = sum(len(j.content or b"") for j in self._jobs.values())
            for jid, j in list(self._jobs.items()):
                if total <= self.store_bytes:
                    break
                if j.content:
                    total -= len(j.content)
                    del self._jobs[jid]

    # ---------------------------------------------------------------- pipeline --
    def _enter(self, job: VideoJob, phase: str) -> None:
        """Phase transition; with ``time_phases`` the device is drained first and the
        wall time of the phase that ends is kept in ``job.timings``."""
        if self.time_phases:
            if self.model.device.type == "cuda":
                torch.cuda.synchronize(self.model.device)
            now = time.perf_counter()
            prev = getattr(job, "_phase_t0", None)
            if prev is not None:
                job.timings[job.phase] = job.timings.get(job.phase, 0.0) + now - prev
            job._phase_t0 = now
        job.phase = phase

    def _keyframe_latents(self, p, lf: int, lh: int, lw: int) -> list:
        """The plan's keyframe and reference images as (latent frame, latent) pairs (frame
        ``None`` for a reference): each image is resized to the clip's raster, normalised and
        encoded alone (a still is one frame).  Every rank encodes the same pixels under the
        same seed, so the latents agree without a copy."""
        if not p.keyframes and not p.references:
            return []
        kind = lambda r: r["type"] if isinstance(r, dict) else r.type
        tracks = [r for r in p.references if kind(r) == "audio"]
        if tracks and self.audio_encoder is None:
            raise ValueError("input_error: input_references: this deployment has no audio "
                             "encoder")
        if self.video_encoder is None:
            raise ValueError("input_error: this deployment has no condition encoder")
        from ..models.h3_vae_encoder import normalize_pixels
        from . import images as IM
        enc, out = self.video_encoder, []
        sp = enc.cfg.spatial
        for frame_index, ref in list(p.keyframes) + [(None, r) for r in p.references]:
            url = ref["url"] if isinstance(ref, dict) else ref.url
            # a clip or a track is read from ``start_time_seconds`` on
            start = float((ref.get("start_time_seconds") if isinstance(ref, dict)
                           else ref.start_time_seconds) or 0.0)
            if start < 0:
                raise ValueError("input_error: input_references: start_time_seconds is negative")
            if frame_index is None and kind(ref) == "audio":
                from ..models.h3_audio_encoder import load_wav, padded_samples
                ac = self.audio_encoder.cfg
                try:
                    wav = load_wav(url, ac.sample_rate)
                except (ValueError, OSError) as e:
                    raise ValueError(f"input_error: input_references: {e}")
                wav = wav[:, :, int(start * ac.sample_rate):][:, :, :int(self.max_seconds *
                                                                         ac.sample_rate)]
                if wav.shape[2] == 0:
                    raise ValueError("input_error: input_references: the track ends before "
                                     "start_time_seconds")
                wav = torch.nn.functional.pad(wav, (0, padded_samples(wav.shape[2], ac.hop) -
                                                    wav.shape[2]))
                self.h2d_bytes += wav.numel() * 4
                out.append((None, self.audio_encoder.encode(wav.to(self.audio_encoder.device))))
                continue
            clip = frame_index is None and kind(ref) == "video"
            try:
                if clip:
                    # frames at the clip's rate, cut to the frame rule (17 n + 5, or one clip
                    # of 17); the soundtrack of a reference clip is not read
                    from .video_rules import FPS
                    skip = int(round(start * FPS))
                    frames, _ = IM.load_video(url, fps=float(FPS),
                                              max_frames=skip + int(self.max_seconds * FPS))
                    frames = frames[skip:]
                    n = (len(frames) - 5) // 17
                    keep = 17 * n + 5 if n >= 1 else 17 if len(frames) >= 17 else 0
                    if keep == 0:
                        raise ValueError("a reference clip has at least 17 frames")
                    rgb = torch.from_numpy(np.ascontiguousarray(frames[:keep])).to(enc.device)
                else:
                    rgb = torch.from_numpy(IM.load_image(url).copy()).to(enc.device)[None]
            except (ValueError, OSError) as e:
                raise ValueError(f"input_error: input_references: {e}")
            self.h2d_bytes += rgb.numel()
            x = rgb.permute(0, 3, 1, 2).float()
            x = torch.nn.functional.interpolate(x, size=(lh * sp, lw * sp), mode="bilinear",
                                                align_corners=False, antialias=True)
            x = normalize_pixels(x.clamp(0, 255).round().to(torch.uint8).permute(0, 2, 3, 1))
            # every 17-frame clip (and the 5-frame tail) is encoded alone
            z = torch.cat([enc.encode_condition(x[:, lo:lo + 17], seed=p.seed)
                           for lo in range(0, x.shape[1], 17)], 1)
            out.append((None if frame_index is None else 0 if frame_index == 0 else lf - 1, z))
        return out

    def generate(self, job: VideoJob) -> bytes:
        cfg, p, dev = self.model.cfg, job.plan, self.model.device
        lf, lh, lw = cfg.latent_shape(p.num_frames, p.width, p.height)
        self._enter(job, "MediaRead")
        conditions = self._keyframe_latents(p, lf, lh, lw)
        self._enter(job, "TextEncode")
        feats = self.text.encode(job.prompt, "cpu")
        if dev.type == "cuda":
            feats = feats.pin_memory().to(dev, non_blocking=True)
            self.h2d_bytes += feats.numel() * feats.element_size()
        self._enter(job, "LatentPrepare")
        n_audio_rows = cfg.audio_rows(p.num_frames)
        st = self.denoiser.prepare(p.seed, lf, lh, lw, n_audio_rows, feats, conditions)
        cap = getattr(getattr(self.model, "ulysses", None), "rows_all", None)
        if cap is not None and st.layout.rows > cap:      # the exchange buffers are sized at start
            raise ValueError(f"input_error: input_references: {st.layout.rows} rows with the "
                             f"conditions, the deployment's exchange buffers hold {cap}")
        saved = self.latent_pool.get(job.id)
        if saved is not None and saved["video"].shape == st.video.shape:
            st.video.copy_(saved["video"].to(st.video.device))
            st.audio.copy_(saved["audio"].to(st.audio.device))
            st.step = saved["step"]
            job.resumed_from = saved["step"]
        self._enter(job, "Denoise")
        while st.step < self.denoiser.steps:
            if job.cancelled:
                raise RuntimeError("cancelled")
            self.denoiser.step(st)
            job.step = st.step
            job.progress = 0.8 * st.step / self.denoiser.steps
            self._save_trajectory(job, st)
        # the audio decoder (rank 0 only needs the samples) starts on a stream of its own and
        # runs beside the video decoder instead of after it
        wav, wav_done = None, None
        if self.rank == 0 and st.audio.is_cuda:
            if self._audio_stream is None:
                self._audio_stream = torch.cuda.Stream(device=st.audio.device)
            self._audio_stream.wait_stream(torch.cuda.current_stream(st.audio.device))
            with torch.cuda.stream(self._audio_stream):
                wav = self._decode_audio(st, cfg, p)
                wav_done = torch.cuda.Event()
                wav_done.record(self._audio_stream)
            st.audio.record_stream(self._audio_stream)
        self._enter(job, "VideoDecode")
        units = self.video_vae.decode(st.video, self.rank, self.world)
        planes = []
        for _, f in units:
            if f.shape[-2:] != (p.height, p.width):
                f = torch.nn.functional.interpolate(f, size=(p.height, p.width),
                                                    mode="bilinear", align_corners=False)
            y, u, v = M.rgb_to_yuv420(f)
            planes.append(torch.cat([y.flatten(1), u.flatten(1), v.flatten(1)], 1))
        packed = self._collect_units(planes, lf, p)
        job.progress = 0.9
        # the planes start their way to (pinned) host memory now, on a copy stream, and land
        # while the audio decoder runs
        host, landed = None, None
        if self.rank == 0 and packed.is_cuda:
            host = self._pinned_planes(packed.shape)
            if self._copy_stream is None:
                self._copy_stream = torch.cuda.Stream(device=packed.device)
            self._copy_stream.wait_stream(torch.cuda.current_stream(packed.device))
            with torch.cuda.stream(self._copy_stream):
                host.copy_(packed, non_blocking=True)
                landed = torch.cuda.Event()
                landed.record(self._copy_stream)
            packed.record_stream(self._copy_stream)
        self._enter(job, "AudioDecode")
        if self.rank != 0:
            return b""
        if wav_done is not None:
            torch.cuda.current_stream(wav.device).wait_event(wav_done)
            wav.record_stream(torch.cuda.current_stream(wav.device))
        else:
            wav = self._decode_audio(st, cfg, p)
        self._enter(job, "VideoEncode")
        hw = p.height * p.width
        if landed is not None:
            landed.synchronize()
        else:
            host = packed.cpu()
        self.d2h_bytes += host.numel()
        y = host[:, :hw].view(-1, p.height, p.width)
        u = host[:, hw:hw + hw // 4].view(-1, p.height // 2, p.width // 2)
        v = host[:, hw + hw // 4:].view(-1, p.height // 2, p.width // 2)
        self._enter(job, "AudioEncode")
        pcm = M.pcm_interleave(wav)
        self.d2h_bytes += pcm.numel() * pcm.element_size()
        self._enter(job, "Mux")
        mp4 = M.write_mp4(y, u, v, p.fps, pcm, self.audio_vae.cfg.sample_rate)
        self._enter(job, "Done")
        return mp4

    def _decode_audio(self, st, cfg, p) -> torch.Tensor:
        """The clip's samples [2, n] from the audio latents (rows are [time x 2 channels,
        latent_channels]: the channels go into the batch), cut or padded to the clip's length."""
        a = st.audio.view(-1, 2, cfg.audio_channels).permute(1, 2, 0).contiguous()
        wav = self.audio_vae.decode(a)
        want = int(round(p.num_frames / p.fps * self.audio_vae.cfg.sample_rate))
        return wav[:, :want] if wav.shape[1] >= want else torch.nn.functional.pad(
            wav, (0, want - wav.shape[1]))

    def _pinned_planes(self, shape) -> torch.Tensor:
        """A pinned host buffer for the packed planes of a clip (kept across requests: pinning
        300 MB costs about as much as the copy it speeds up)."""
        n = 1
        for d in shape:
            n *= int(d)
        if self._pinned is None or self._pinned.numel() < n:
            self._pinned = torch.empty(n, dtype=torch.uint8, pin_memory=True)
        return self._pinned[:n].view(*shape)

    def _collect_units(self, planes: list, latent_frames: int, p) -> torch.Tensor:
        """Packed 4:2:0 planes of every frame in order, [frames, 1.5 * H * W] uint8.
        Under a sequence group each rank encoded its own temporal units; the
        blocks are all-gathered (padded to the largest share) and put in order."""
        width = p.height * p.width * 3 // 2
        dev = self.model.device
        own = torch.cat(planes, 0) if planes else torch.empty(0, width, dtype=torch.uint8,
                                                                device=dev)
        if self.world == 1:
            return own[:p.num_frames]
        import torch.distributed as dist
        unit = 5
        n_units = (latent_frames + unit - 1) // unit
        T = self.video_vae.cfg.temporal

        def frames_of(k):   # frames unit k produces
            f = min(unit, latent_frames - k * unit)
            return 1 + T * (f - 1)
        share = [sum(frames_of(k) for k in range(r, n_units, self.world))
                 for r in range(self.world)]
        cap = max(share)
        buf = torch.zeros(cap, width, dtype=torch.uint8, device=dev)
        buf[:own.shape[0]] = own
        allb = torch.empty(self.world * cap, width, dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(allb, buf, group=self.group)
        allb = allb.view(self.world, cap, width)
        cursor = [0] * self.world
        out = []
        for k in range(n_units):
            r, n = k % self.world, frames_of(k)
            out.append(allb[r, cursor[r]:cursor[r] + n])
            cursor[r] += n
        return torch.cat(out, 0)[:p.num_frames]

    def _save_trajectory(self, job: VideoJob, st) -> None:
        if st.step >= self.denoiser.steps:
            self.latent_pool.pop(job.id, None)          # nothing left to resume
            return
        ent = {"step": st.step, "video": st.video.detach().to("cpu", copy=True),
               "audio": st.audio.detach().to("cpu", copy=True)}
        self.d2h_bytes += ent["video"].numel() * 4 + ent["audio"].numel() * 4
        self.latent_pool[job.id] = ent
        self.latent_pool.move_to_end(job.id)
        size = lambda e: (e["video"].numel() + e["audio"].numel()) * 4
        while sum(size(e) for e in self.latent_pool.values()) > self.latent_pool_bytes and \
                len(self.latent_pool) > 1:
            self.latent_pool.popitem(last=False)

    def resume(self, job_id: str) -> bool:
        """Queues a failed job again; it continues from its last saved step boundary."""
        with self._cv:
            job = self._jobs.get(job_id)
            if job is None or job.state != "failed" or job.cancelled:
                return False
            job.state, job.error, job.completed_at = "queued", None, None
            job._done.clear()
            self._queue.append(job)
            self._cv.notify_all()
        return True

    def _run(self):
        while True:
            with self._cv:
                while not self._queue and not self._stop:
                    self._cv.wait(0.5)
                if self._stop:
                    return
                job = self._queue.pop(0)
            job.state = "in_progress"
            t0 = time.monotonic()
            try:
                job.content = self.generate(job)
                job.progress = 1.0
                job.finish("completed")
                if self.obs:
                    self.obs.observe("uniserve_video_seconds", time.monotonic() - t0)
                    self.obs.inc("uniserve_requests_total", {"outcome": "completed"})
            except Exception as e:
                # a failure inside the trajectory is retried from the last boundary
                if not job.cancelled and job.id in self.latent_pool and \
                        job.resumes < self.max_resumes:
                    job.resumes += 1
                    with self._cv:
                        self._queue.insert(0, job)
                    continue
                self.latent_pool.pop(job.id, None)
                job.finish("failed", str(e))
                if self.obs:
                    self.obs.inc("uniserve_requests_total", {"outcome": "failed"})
