// Host-side media output: H.264 elementary stream + MP4 (ISO BMFF) muxer + WAV.
//
// Neither FFmpeg nor libx264 exists on the target image, so the encoder here is a
// self-contained H.264 writer that emits a conforming Constrained Baseline stream
// made of IDR pictures whose macroblocks are all I_PCM (raw 4:2:0 samples): every
// decoder plays it, nothing is lost, nothing is compressed.  The audio track is
// 16-bit PCM ('ipcm' sample entry, ISO/IEC 23003-5) because no AAC encoder is
// available either.  The reference encodes with libx264 (ultrafast / zerolatency)
// and AAC through its FFmpeg shim (crates/media/src/ffi/shim.c, crates/media/src/lib.rs:39-45,
// reference project paths); the container layout (one video track of 24 fps
// frames, one 32 kHz audio track, moov after mdat) follows the same contract.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>
#include <thread>
#include <algorithm>

#define US_API extern "C" __attribute__((visibility("default")))

namespace {

struct Bits {
  std::vector<uint8_t> buf;
  uint32_t cur = 0;
  int n = 0;
  void put(uint32_t v, int bits) {
    for (int i = bits - 1; i >= 0; --i) {
      cur = (cur << 1) | ((v >> i) & 1u);
      if (++n == 8) {
        buf.push_back((uint8_t)cur);
        cur = 0;
        n = 0;
      }
    }
  }
  void ue(uint32_t v) {
    const uint32_t x = v + 1;
    int len = 0;
    while ((x >> len) > 1) ++len;
    put(0, len);
    put(x, len + 1);
  }
  void se(int v) { ue(v <= 0 ? (uint32_t)(-2 * v) : (uint32_t)(2 * v - 1)); }
  bool aligned() const { return n == 0; }
  void align_zero() {
    while (n) put(0, 1);
  }
  void trailing() {
    put(1, 1);
    align_zero();
  }
  void bytes(const uint8_t* p, size_t len) { buf.insert(buf.end(), p, p + len); }
};

// Adds emulation prevention and the NAL header; returns the NAL unit (no start code).
std::vector<uint8_t> nal(uint8_t ref_idc, uint8_t type, const std::vector<uint8_t>& rbsp) {
  std::vector<uint8_t> out;
  out.reserve(rbsp.size() + rbsp.size() / 64 + 8);
  out.push_back((uint8_t)((ref_idc << 5) | type));
  int zeros = 0;
  for (uint8_t b : rbsp) {
    if (zeros >= 2 && b <= 3) {
      out.push_back(3);
      zeros = 0;
    }
    out.push_back(b);
    zeros = (b == 0) ? zeros + 1 : 0;
  }
  return out;
}

std::vector<uint8_t> make_sps(int width, int height) {
  const int mbw = (width + 15) / 16, mbh = (height + 15) / 16;
  Bits b;
  b.put(66, 8);        // profile_idc: Baseline
  b.put(0xC0, 8);      // constraint_set0/1 flags (Constrained Baseline)
  b.put(51, 8);        // level_idc 5.1
  b.ue(0);             // seq_parameter_set_id
  b.ue(0);             // log2_max_frame_num_minus4
  b.ue(2);             // pic_order_cnt_type 2: output order = decoding order
  b.ue(0);             // max_num_ref_frames
  b.put(0, 1);         // gaps_in_frame_num_value_allowed_flag
  b.ue(mbw - 1);
  b.ue(mbh - 1);
  b.put(1, 1);         // frame_mbs_only_flag
  b.put(0, 1);         // direct_8x8_inference_flag
  const int cr = mbw * 16 - width, cb = mbh * 16 - height;
  if (cr || cb) {
    b.put(1, 1);
    b.ue(0);
    b.ue(cr / 2);
    b.ue(0);
    b.ue(cb / 2);
  } else {
    b.put(0, 1);
  }
  b.put(0, 1);         // vui_parameters_present_flag
  b.trailing();
  return b.buf;
}

std::vector<uint8_t> make_pps() {
  Bits b;
  b.ue(0);             // pic_parameter_set_id
  b.ue(0);             // seq_parameter_set_id
  b.put(0, 1);         // entropy_coding_mode_flag: CAVLC
  b.put(0, 1);         // bottom_field_pic_order_in_frame_present_flag
  b.ue(0);             // num_slice_groups_minus1
  b.ue(0);             // num_ref_idx_l0_default_active_minus1
  b.ue(0);             // num_ref_idx_l1_default_active_minus1
  b.put(0, 1);         // weighted_pred_flag
  b.put(0, 2);         // weighted_bipred_idc
  b.se(0);             // pic_init_qp_minus26
  b.se(0);             // pic_init_qs_minus26
  b.se(0);             // chroma_qp_index_offset
  b.put(1, 1);         // deblocking_filter_control_present_flag
  b.put(0, 1);         // constrained_intra_pred_flag
  b.put(0, 1);         // redundant_pic_cnt_present_flag
  b.trailing();
  return b.buf;
}

// One IDR picture, every macroblock I_PCM.
std::vector<uint8_t> make_idr(const uint8_t* y, const uint8_t* u, const uint8_t* v, int width,
                              int height, int idr_id) {
  const int mbw = (width + 15) / 16, mbh = (height + 15) / 16;
  Bits b;
  b.buf.reserve((size_t)mbw * mbh * 386 + 64);
  b.ue(0);             // first_mb_in_slice
  b.ue(7);             // slice_type: I (all slices of the picture)
  b.ue(0);             // pic_parameter_set_id
  b.put(0, 4);         // frame_num
  b.ue(idr_id & 0xFFFF);
  b.put(0, 1);         // no_output_of_prior_pics_flag
  b.put(0, 1);         // long_term_reference_flag
  b.se(0);             // slice_qp_delta
  b.ue(1);             // disable_deblocking_filter_idc: off
  uint8_t mb[384];
  for (int my = 0; my < mbh; ++my)
    for (int mx = 0; mx < mbw; ++mx) {
      b.ue(25);        // mb_type I_PCM
      b.align_zero();  // pcm_alignment_zero_bit
      const int cw = width / 2, ch = height / 2;
      if (mx * 16 + 16 <= width && my * 16 + 16 <= height) {
        // a macroblock inside the picture: whole rows at a time
        for (int r = 0; r < 16; ++r)
          memcpy(mb + r * 16, y + (size_t)(my * 16 + r) * width + mx * 16, 16);
        for (int r = 0; r < 8; ++r) {
          memcpy(mb + 256 + r * 8, u + (size_t)(my * 8 + r) * cw + mx * 8, 8);
          memcpy(mb + 320 + r * 8, v + (size_t)(my * 8 + r) * cw + mx * 8, 8);
        }
      } else {                                   // the picture's edge is repeated
        for (int r = 0; r < 16; ++r) {
          const int yy = my * 16 + r < height ? my * 16 + r : height - 1;
          for (int c = 0; c < 16; ++c) {
            const int xx = mx * 16 + c < width ? mx * 16 + c : width - 1;
            mb[r * 16 + c] = y[(size_t)yy * width + xx];
          }
        }
        for (int r = 0; r < 8; ++r) {
          const int yy = my * 8 + r < ch ? my * 8 + r : ch - 1;
          for (int c = 0; c < 8; ++c) {
            const int xx = mx * 8 + c < cw ? mx * 8 + c : cw - 1;
            mb[256 + r * 8 + c] = u[(size_t)yy * cw + xx];
            mb[320 + r * 8 + c] = v[(size_t)yy * cw + xx];
          }
        }
      }
      b.bytes(mb, 384);
    }
  b.trailing();
  return nal(3, 5, b.buf);
}

// ------------------------------------------------------------------ MP4 boxes --
struct Box {
  std::vector<uint8_t> d;
  void u8(uint32_t v) { d.push_back((uint8_t)v); }
  void u16(uint32_t v) { u8(v >> 8); u8(v); }
  void u32(uint32_t v) { u16(v >> 16); u16(v); }
  void u64(uint64_t v) { u32((uint32_t)(v >> 32)); u32((uint32_t)v); }
  void str(const char* s, size_t n) { d.insert(d.end(), s, s + n); }
  void zeros(size_t n) { d.insert(d.end(), n, 0); }
  void add(const Box& b) { d.insert(d.end(), b.d.begin(), b.d.end()); }
};
Box box(const char* type, const Box& payload) {
  Box b;
  b.u32((uint32_t)payload.d.size() + 8);
  b.str(type, 4);
  b.add(payload);
  return b;
}
Box full(uint8_t version, uint32_t flags) {
  Box b;
  b.u32(((uint32_t)version << 24) | flags);
  return b;
}
void matrix(Box& b) {
  const uint32_t m[9] = {0x10000, 0, 0, 0, 0x10000, 0, 0, 0, 0x40000000};
  for (uint32_t v : m) b.u32(v);
}

struct Track {
  bool video;
  uint32_t id, timescale;
  uint64_t duration;                    // in timescale units
  std::vector<uint32_t> sample_sizes;   // video: per frame; audio: empty (uniform)
  uint32_t uniform_size = 0, sample_count = 0, sample_delta = 1;
  std::vector<uint64_t> chunk_offsets;
  uint32_t samples_per_chunk = 1;
  int width = 0, height = 0, channels = 0, sample_rate = 0;
  std::vector<uint8_t> sps, pps;
};

Box stbl(const Track& t) {
  Box entry;
  if (t.video) {
    Box e;
    e.zeros(6); e.u16(1);               // reserved, data_reference_index
    e.zeros(16);
    e.u16(t.width); e.u16(t.height);
    e.u32(0x00480000); e.u32(0x00480000);
    e.u32(0); e.u16(1);
    e.zeros(32);                        // compressorname
    e.u16(0x18); e.u16(0xFFFF);
    Box c;
    c.u8(1); c.u8(t.sps[1]); c.u8(t.sps[2]); c.u8(t.sps[3]);
    c.u8(0xFF);                         // 4-byte NAL lengths
    c.u8(0xE1); c.u16((uint32_t)t.sps.size()); c.d.insert(c.d.end(), t.sps.begin(), t.sps.end());
    c.u8(1); c.u16((uint32_t)t.pps.size()); c.d.insert(c.d.end(), t.pps.begin(), t.pps.end());
    e.add(box("avcC", c));
    entry = box("avc1", e);
  } else {
    Box e;
    e.zeros(6); e.u16(1);
    e.zeros(8);
    e.u16(t.channels); e.u16(16); e.u32(0);
    e.u32((uint32_t)t.sample_rate << 16);
    Box p = full(0, 0);
    p.u8(1);                            // format_flags: little endian
    p.u8(16);                           // PCM_sample_size
    e.add(box("pcmC", p));
    entry = box("ipcm", e);
  }
  Box stsd = full(0, 0);
  stsd.u32(1);
  stsd.add(entry);
  Box stts = full(0, 0);
  stts.u32(1); stts.u32(t.sample_count); stts.u32(t.sample_delta);
  Box stsc = full(0, 0);
  stsc.u32(1); stsc.u32(1); stsc.u32(t.samples_per_chunk); stsc.u32(1);
  Box stsz = full(0, 0);
  stsz.u32(t.uniform_size); stsz.u32(t.sample_count);
  if (!t.uniform_size) for (uint32_t s : t.sample_sizes) stsz.u32(s);
  Box co64 = full(0, 0);
  co64.u32((uint32_t)t.chunk_offsets.size());
  for (uint64_t o : t.chunk_offsets) co64.u64(o);
  Box s;
  s.add(box("stsd", stsd)); s.add(box("stts", stts));
  if (t.video) {                        // every sample is a sync sample: no stss needed
  }
  s.add(box("stsc", stsc)); s.add(box("stsz", stsz)); s.add(box("co64", co64));
  return box("stbl", s);
}

Box trak(const Track& t, uint32_t movie_timescale) {
  Box tkhd = full(0, 3);
  tkhd.u32(0); tkhd.u32(0); tkhd.u32(t.id); tkhd.u32(0);
  tkhd.u32((uint32_t)(t.duration * movie_timescale / t.timescale));
  tkhd.zeros(8); tkhd.u16(0); tkhd.u16(0); tkhd.u16(t.video ? 0 : 0x0100); tkhd.u16(0);
  matrix(tkhd);
  tkhd.u32((uint32_t)t.width << 16); tkhd.u32((uint32_t)t.height << 16);
  Box mdhd = full(0, 0);
  mdhd.u32(0); mdhd.u32(0); mdhd.u32(t.timescale); mdhd.u32((uint32_t)t.duration);
  mdhd.u16(0x55C4); mdhd.u16(0);
  Box hdlr = full(0, 0);
  hdlr.u32(0); hdlr.str(t.video ? "vide" : "soun", 4); hdlr.zeros(12);
  hdlr.str(t.video ? "VideoHandler" : "SoundHandler", 13);
  Box mh = t.video ? full(0, 1) : full(0, 0);
  if (t.video) mh.zeros(8); else mh.zeros(4);
  Box url = full(0, 1);
  Box dref = full(0, 0);
  dref.u32(1); dref.add(box("url ", url));
  Box dinf;
  dinf.add(box("dref", dref));
  Box minf;
  minf.add(box(t.video ? "vmhd" : "smhd", mh)); minf.add(box("dinf", dinf)); minf.add(stbl(t));
  Box mdia;
  mdia.add(box("mdhd", mdhd)); mdia.add(box("hdlr", hdlr)); mdia.add(box("minf", minf));
  Box tr;
  tr.add(box("tkhd", tkhd)); tr.add(box("mdia", mdia));
  return box("trak", tr);
}

}  // namespace

// Annex-B elementary stream (start codes) of n frames; returns bytes written or -1.
US_API long long us_h264_encode_annexb(const char* path, int width, int height, int n_frames,
                                       const uint8_t* y, const uint8_t* u, const uint8_t* v) {
  FILE* f = fopen(path, "wb");
  if (!f) return -1;
  const uint8_t sc[4] = {0, 0, 0, 1};
  long long total = 0;
  auto emit = [&](const std::vector<uint8_t>& n) {
    fwrite(sc, 1, 4, f);
    fwrite(n.data(), 1, n.size(), f);
    total += 4 + (long long)n.size();
  };
  emit(nal(3, 7, make_sps(width, height)));
  emit(nal(3, 8, make_pps()));
  const size_t ys = (size_t)width * height, cs = ys / 4;
  for (int i = 0; i < n_frames; ++i) emit(make_idr(y + i * ys, u + i * cs, v + i * cs, width, height, i));
  fclose(f);
  return total;
}

// MP4 with one H.264 video track (fps frames per second) and, when pcm != NULL, one
// 16-bit PCM audio track.  Planes are contiguous per frame.  Returns bytes written or -1.
US_API long long us_mp4_write(const char* path, int width, int height, int fps, int n_frames,
                              const uint8_t* y, const uint8_t* u, const uint8_t* v,
                              const int16_t* pcm, long long audio_frames, int channels,
                              int sample_rate) {
  if (!path || width < 16 || height < 16 || (width & 1) || (height & 1) || fps < 1 ||
      n_frames < 1 || !y || !u || !v)
    return -1;
  FILE* f = fopen(path, "wb");
  if (!f) return -1;
  Box ft;
  ft.str("isom", 4); ft.u32(0x200); ft.str("isomiso2avc1mp41", 16);
  Box ftyp = box("ftyp", ft);
  fwrite(ftyp.d.data(), 1, ftyp.d.size(), f);
  uint64_t pos = ftyp.d.size();
  // mdat with a 64-bit size, patched at the end
  const uint64_t mdat_at = pos;
  const uint8_t hdr[16] = {0, 0, 0, 1, 'm', 'd', 'a', 't'};
  fwrite(hdr, 1, 16, f);
  pos += 16;
  Track vt;
  vt.video = true; vt.id = 1; vt.timescale = (uint32_t)fps * 512; vt.sample_delta = 512;
  vt.width = width; vt.height = height;
  vt.sps = nal(3, 7, make_sps(width, height));
  vt.pps = nal(3, 8, make_pps());
  const size_t ys = (size_t)width * height, cs = ys / 4;
  // Pictures are independent (every one is an IDR): build them on several threads,
  // a window at a time, and write them in order.
  const int workers = std::max(1, std::min({(int)std::thread::hardware_concurrency(), 16,
                                            n_frames}));
  std::vector<std::vector<uint8_t>> window(workers);
  for (int i = 0; i < n_frames; ++i) {
    if (i % workers == 0) {
      std::vector<std::thread> pool;
      const int n = std::min(workers, n_frames - i);
      for (int t = 0; t < n; ++t)
        pool.emplace_back([&, t] {
          const int fi = i + t;
          window[t] = make_idr(y + fi * ys, u + fi * cs, v + fi * cs, width, height, fi);
        });
      for (auto& th : pool) th.join();
    }
    const std::vector<uint8_t>& au = window[i % workers];
    const uint32_t len = (uint32_t)au.size();
    const uint8_t l4[4] = {(uint8_t)(len >> 24), (uint8_t)(len >> 16), (uint8_t)(len >> 8),
                           (uint8_t)len};
    vt.chunk_offsets.push_back(pos);
    fwrite(l4, 1, 4, f);
    fwrite(au.data(), 1, au.size(), f);
    vt.sample_sizes.push_back(len + 4);
    pos += len + 4;
  }
  vt.sample_count = (uint32_t)n_frames;
  vt.duration = (uint64_t)n_frames * 512;
  Track at;
  const bool audio = pcm != nullptr && audio_frames > 0 && channels >= 1;
  if (audio) {
    at.video = false; at.id = 2; at.timescale = (uint32_t)sample_rate; at.sample_delta = 1;
    at.channels = channels; at.sample_rate = sample_rate;
    at.uniform_size = (uint32_t)(2 * channels);
    at.sample_count = (uint32_t)audio_frames;
    at.samples_per_chunk = (uint32_t)audio_frames;
    at.chunk_offsets.push_back(pos);
    at.duration = (uint64_t)audio_frames;
    fwrite(pcm, 2 * (size_t)channels, (size_t)audio_frames, f);
    pos += 2ull * channels * audio_frames;
  }
  const uint64_t mdat_size = pos - mdat_at;
  const uint32_t movie_ts = 1000;
  Box mvhd = full(0, 0);
  mvhd.u32(0); mvhd.u32(0); mvhd.u32(movie_ts);
  mvhd.u32((uint32_t)((uint64_t)n_frames * movie_ts / fps));
  mvhd.u32(0x10000); mvhd.u16(0x0100); mvhd.zeros(10);
  matrix(mvhd);
  mvhd.zeros(24);
  mvhd.u32(audio ? 3 : 2);
  Box moov;
  moov.add(box("mvhd", mvhd));
  moov.add(trak(vt, movie_ts));
  if (audio) moov.add(trak(at, movie_ts));
  Box mv = box("moov", moov);
  fwrite(mv.d.data(), 1, mv.d.size(), f);
  pos += mv.d.size();
  fseek(f, (long)mdat_at + 8, SEEK_SET);
  uint8_t sz[8];
  for (int i = 0; i < 8; ++i) sz[i] = (uint8_t)(mdat_size >> (56 - 8 * i));
  fwrite(sz, 1, 8, f);
  fclose(f);
  return (long long)pos;
}

// The same MP4 built in memory, in two calls so that the caller can allocate the exact size:
// us_mp4_build encodes every picture (one thread slot each) and lays the file out, returning a
// handle and the size; us_mp4_take copies the file into the caller's buffer (pictures in
// parallel) and frees the handle.  No file round trip, no oversized scratch buffer.
struct Mp4Built {
  std::vector<uint8_t> head;                    // ftyp + mdat header
  std::vector<std::vector<uint8_t>> pics;
  std::vector<uint64_t> at_pos;
  const int16_t* pcm = nullptr;
  uint64_t audio_at = 0, audio_bytes = 0, moov_at = 0, total = 0;
  std::vector<uint8_t> moov;
  int workers = 1;
};

US_API void* us_mp4_build(int width, int height, int fps, int n_frames, const uint8_t* y,
                          const uint8_t* u, const uint8_t* v, const int16_t* pcm,
                          long long audio_frames, int channels, int sample_rate,
                          long long* size_out) {
  if (width < 16 || height < 16 || (width & 1) || (height & 1) || fps < 1 || n_frames < 1 ||
      !y || !u || !v || !size_out)
    return nullptr;
  Mp4Built* b = new Mp4Built();
  Box ft;
  ft.str("isom", 4); ft.u32(0x200); ft.str("isomiso2avc1mp41", 16);
  Box ftyp = box("ftyp", ft);
  const size_t ys = (size_t)width * height, cs = ys / 4;
  b->workers = std::max(1, std::min({(int)std::thread::hardware_concurrency(), 32, n_frames}));
  b->pics.resize(n_frames);
  {
    std::vector<std::thread> pool;
    for (int t = 0; t < b->workers; ++t)
      pool.emplace_back([&, t] {
        for (int fi = t; fi < n_frames; fi += b->workers)
          b->pics[fi] = make_idr(y + fi * ys, u + fi * cs, v + fi * cs, width, height, fi);
      });
    for (auto& th : pool) th.join();
  }
  Track vt;
  vt.video = true; vt.id = 1; vt.timescale = (uint32_t)fps * 512; vt.sample_delta = 512;
  vt.width = width; vt.height = height;
  vt.sps = nal(3, 7, make_sps(width, height));
  vt.pps = nal(3, 8, make_pps());
  uint64_t pos = ftyp.d.size();
  const uint64_t mdat_at = pos;
  pos += 16;
  b->at_pos.resize(n_frames);
  for (int i = 0; i < n_frames; ++i) {
    b->at_pos[i] = pos;
    vt.chunk_offsets.push_back(pos);
    vt.sample_sizes.push_back((uint32_t)b->pics[i].size() + 4);
    pos += b->pics[i].size() + 4;
  }
  vt.sample_count = (uint32_t)n_frames;
  vt.duration = (uint64_t)n_frames * 512;
  Track at;
  const bool audio = pcm != nullptr && audio_frames > 0 && channels >= 1;
  b->audio_at = pos;
  if (audio) {
    at.video = false; at.id = 2; at.timescale = (uint32_t)sample_rate; at.sample_delta = 1;
    at.channels = channels; at.sample_rate = sample_rate;
    at.uniform_size = (uint32_t)(2 * channels);
    at.sample_count = (uint32_t)audio_frames;
    at.samples_per_chunk = (uint32_t)audio_frames;
    at.chunk_offsets.push_back(pos);
    at.duration = (uint64_t)audio_frames;
    b->pcm = pcm;
    b->audio_bytes = 2ull * channels * audio_frames;
    pos += b->audio_bytes;
  }
  const uint64_t mdat_size = pos - mdat_at;
  const uint32_t movie_ts = 1000;
  Box mvhd = full(0, 0);
  mvhd.u32(0); mvhd.u32(0); mvhd.u32(movie_ts);
  mvhd.u32((uint32_t)((uint64_t)n_frames * movie_ts / fps));
  mvhd.u32(0x10000); mvhd.u16(0x0100); mvhd.zeros(10);
  matrix(mvhd);
  mvhd.zeros(24);
  mvhd.u32(audio ? 3 : 2);
  Box moov;
  moov.add(box("mvhd", mvhd));
  moov.add(trak(vt, movie_ts));
  if (audio) moov.add(trak(at, movie_ts));
  Box mv = box("moov", moov);
  b->moov = mv.d;
  b->moov_at = pos;
  b->total = pos + mv.d.size();
  b->head = ftyp.d;
  uint8_t hdr[16] = {0, 0, 0, 1, 'm', 'd', 'a', 't'};
  for (int i = 0; i < 8; ++i) hdr[8 + i] = (uint8_t)(mdat_size >> (56 - 8 * i));
  b->head.insert(b->head.end(), hdr, hdr + 16);
  *size_out = (long long)b->total;
  return b;
}

// Copies the built file into `out` (at least the size us_mp4_build reported; the audio samples
// passed to us_mp4_build must still be alive) and frees the handle.  `out` may be null to
// discard the handle.
US_API long long us_mp4_take(void* handle, uint8_t* out) {
  if (!handle) return -1;
  Mp4Built* b = (Mp4Built*)handle;
  const long long total = (long long)b->total;
  if (out) {
    memcpy(out, b->head.data(), b->head.size());
    const int n_frames = (int)b->pics.size();
    std::vector<std::thread> pool;
    for (int t = 0; t < b->workers; ++t)
      pool.emplace_back([&, t] {
        for (int fi = t; fi < n_frames; fi += b->workers) {
          const uint32_t len = (uint32_t)b->pics[fi].size();
          uint8_t* d = out + b->at_pos[fi];
          d[0] = (uint8_t)(len >> 24); d[1] = (uint8_t)(len >> 16);
          d[2] = (uint8_t)(len >> 8); d[3] = (uint8_t)len;
          memcpy(d + 4, b->pics[fi].data(), len);
        }
      });
    for (auto& th : pool) th.join();
    if (b->audio_bytes) memcpy(out + b->audio_at, b->pcm, b->audio_bytes);
    memcpy(out + b->moov_at, b->moov.data(), b->moov.size());
  }
  delete b;
  return total;
}

US_API long long us_wav_write(const char* path, const int16_t* pcm, long long frames, int channels,
                              int sample_rate) {
  FILE* f = fopen(path, "wb");
  if (!f) return -1;
  const uint32_t data = (uint32_t)(frames * channels * 2);
  auto w32 = [&](uint32_t v) { fwrite(&v, 4, 1, f); };
  auto w16 = [&](uint16_t v) { fwrite(&v, 2, 1, f); };
  fwrite("RIFF", 1, 4, f); w32(36 + data); fwrite("WAVEfmt ", 1, 8, f);
  w32(16); w16(1); w16((uint16_t)channels); w32((uint32_t)sample_rate);
  w32((uint32_t)(sample_rate * channels * 2)); w16((uint16_t)(channels * 2)); w16(16);
  fwrite("data", 1, 4, f); w32(data);
  fwrite(pcm, 2, (size_t)frames * channels, f);
  fclose(f);
  return 44 + (long long)data;
}
