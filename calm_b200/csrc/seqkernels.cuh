// seqkernels.cuh -- device code of the layer-list models (include/calm_b200_seq.h): packed batches of tokens from many
// sequences, a paged cache for what is indexed by position and per-slot buffers for what is recurrent.
//
// Precision: the residual stream, every norm, softmax, the convolution state, the recurrent state and everything that
// feeds the recurrence after the projections are fp32.  Products read activations of type AT: float (exact mode, SIMT
// FMA) or bf16 (tensor cores, fp32 accumulation).  Weights are bf16 as stored.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"

typedef __nv_bfloat16 bf16;

// per-step description of the packed batch (device arrays)
struct SeqBatch {
	const int* tok;      // [N] token ids
	const int* tslot;    // [N] slot of the token's sequence
	const int* tpos;     // [N] position of the token in its sequence
	const int* tfirst;   // [N] packed index of the first token its sequence has in this step
	const int* sstart;   // [B] first packed index of sequence b
	const int* scount;   // [B]
	const int* spos0;    // [B] position of its first new token
	const int* sslot;    // [B]
	const int* pages;    // [slots][max_pages] page table
	int N, B, max_pages, page;
};

__device__ __forceinline__ long cache_row(const SeqBatch& sb, int slot, int pos) {
	return (long)sb.pages[(long)slot * sb.max_pages + pos / sb.page] * sb.page + pos % sb.page;
}

template <typename T>
__device__ __forceinline__ T to_act(float v);
template <>
__device__ __forceinline__ float to_act<float>(float v) {
	return v;
}
template <>
__device__ __forceinline__ bf16 to_act<bf16>(float v) {
	return __float2bfloat16_rn(v);
}
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float ldf(const float* p) { return *p; }

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }
// warp_sum / warp_max: common.cuh

// ---------------------------------------------------------------- embedding, norms, small element-wise kernels

// x[n] = E[tok[n]] * scale (+ P[position of n], a learned position row, not scaled), written to every one of `streams` copies
// (and a second copy when a looped span re-adds the embedding).  With a bigram table, row (previous token * mul_prev + token * mul_cur)
// mod buckets of it is added as well; a sequence's first token (tprev < 0) takes row `buckets`, the table's last.
struct EmbedBigram {
	const bf16* table; // (buckets + 1, width) or null
	const int* tprev;  // [N] the token before each packed token in its sequence, -1 for a first token
	int buckets, mul_prev, mul_cur;
};
__global__ void k_seq_embed(float* x, float* x0, const bf16* table, const int* tok, int N, int width, float scale, const bf16* pos_table, const int* tpos, int streams, EmbedBigram bg) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const int n = blockIdx.x;
	const bf16* e = table + (size_t)tok[n] * width;
	const bf16* pr = pos_table ? pos_table + (size_t)tpos[n] * width : nullptr;
	const bf16* br = nullptr;
	if (bg.table) {
		const int prev = bg.tprev[n];
		const long long row = prev < 0 ? bg.buckets : ((long long)prev * bg.mul_prev + (long long)tok[n] * bg.mul_cur) % bg.buckets;
		br = bg.table + (size_t)row * width;
	}
	for (int i = threadIdx.x; i < width; i += blockDim.x) {
		float v = ldf(e + i) * scale;
		if (pr) v += ldf(pr + i);
		if (br) v += ldf(br + i);
		for (int s = 0; s < streams; ++s) x[((size_t)n * streams + s) * width + i] = v;
		if (x0) x0[(size_t)n * width + i] = v;
	}
}

__global__ void k_seq_add(float* x, const float* y, size_t n) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i < n) x[i] += y[i];
}

// Dynamic Tanh: out[r][i] = tanh(alpha * x[rows ? rows[r] : r][i]) * w[i] + b[i]
template <typename AT>
__global__ void k_seq_dyt(AT* out, const float* x, const int* rows, const bf16* w, const bf16* b, const bf16* alpha, int R, int width) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= (size_t)R * width) return;
	const int r = (int)(i / width), c = (int)(i % width);
	const float a = ldf(alpha);
	const size_t src = (size_t)(rows ? rows[r] : r) * width + c;
	out[i] = to_act<AT>(tanhf(a * x[src]) * ldf(w + c) + ldf(b + c));
}

// RMS norm of whole rows: out[r][i] = x[row][i] / sqrt(mean(x[row]^2) + eps) * (w[i] + offset); one CTA per row (a single decoded
// token of a wide model is one row: a warp alone would walk it in a hundred dependent steps), the row is read once (up to
// blockDim * RMS_KEEP columns stay in registers, wider rows are read a second time)
#define RMS_KEEP 16
template <typename AT>
__global__ void __launch_bounds__(256) k_seq_rms(AT* out, const float* x, const int* rows, const bf16* w, float offset, float eps, int R, int width) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	__shared__ float red[8];
	const int tid = threadIdx.x, nt = blockDim.x, r = blockIdx.x;
	const float* src = x + (size_t)(rows ? rows[r] : r) * width;
	float keep[RMS_KEEP];
	float ss = 0.f;
#pragma unroll
	for (int i = 0; i < RMS_KEEP; ++i) {
		const int c = i * nt + tid;
		keep[i] = c < width ? src[c] : 0.f;
		ss = fmaf(keep[i], keep[i], ss);
	}
	for (int c = RMS_KEEP * nt + tid; c < width; c += nt) ss = fmaf(src[c], src[c], ss);
	ss = warp_sum(ss);
	if ((tid & 31) == 0) red[tid >> 5] = ss;
	__syncthreads();
	ss = 0.f;
	for (int i = 0; i < (nt >> 5); ++i) ss += red[i]; // every thread adds the warps' sums in the same order
	const float rinv = 1.f / sqrtf(ss / (float)width + eps);
	AT* d = out + (size_t)r * width;
#pragma unroll
	for (int i = 0; i < RMS_KEEP; ++i) {
		const int c = i * nt + tid;
		if (c < width) d[c] = to_act<AT>(keep[i] * rinv * (ldf(w + c) + offset));
	}
	for (int c = RMS_KEEP * nt + tid; c < width; c += nt) d[c] = to_act<AT>(src[c] * rinv * (ldf(w + c) + offset));
}

// RMS norm with a weight over `len` columns of src rows: segment s of blockIdx.y.  Segment 0 goes to an activation
// matrix, segment 1 (the cached latent) to its cache row.
struct RmsSeg {
	int col, len;
	const bf16* w;
};
template <typename AT>
__global__ void k_seq_latent_norm(const float* proj, int ldp, RmsSeg sq, RmsSeg sc, AT* cq, float* cache, SeqBatch sb, float eps) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int n = blockIdx.x * (blockDim.x >> 5) + warp;
	if (n >= sb.N) return;
	const RmsSeg s = blockIdx.y ? sc : sq;
	const float* src = proj + (size_t)n * ldp + s.col;
	float ss = 0.f;
	for (int i = lane; i < s.len; i += 32) ss += src[i] * src[i];
	ss = warp_sum(ss);
	const float r = 1.f / sqrtf(ss / (float)s.len + eps);
	if (blockIdx.y == 0) {
		AT* d = cq + (size_t)n * s.len;
		for (int i = lane; i < s.len; i += 32) d[i] = to_act<AT>(src[i] * r * ldf(s.w + i));
	} else {
		float* d = cache + cache_row(sb, sb.tslot[n], sb.tpos[n]) * s.len;
		for (int i = lane; i < s.len; i += 32) d[i] = src[i] * r * ldf(s.w + i);
	}
}

// copy `len` columns of fp32 rows into an activation matrix
template <typename AT>
__global__ void k_seq_cast_cols(AT* out, const float* src, int lds, int col, int len, int N) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= (size_t)N * len) return;
	out[i] = to_act<AT>(src[(i / len) * lds + col + i % len]);
}

// queries for the product path with fp32-accurate scores: per (token, head) the row [hi | hi | lo] of bf16 values, hi = bf16(q), lo = bf16(q - hi);
// against key rows [hi | lo | hi] one product of depth 3 kd sums q_hi k_hi + q_hi k_lo + q_lo k_hi in fp32
__global__ void k_seq_split_q(bf16* out, const float* q, int kd, size_t units) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= units * kd) return;
	const size_t u = i / kd, d = i % kd;
	const float v = q[i];
	const bf16 hi = __float2bfloat16_rn(v);
	bf16* r = out + u * 3 * kd;
	r[d] = hi, r[kd + d] = hi, r[2 * kd + d] = __float2bfloat16_rn(v - __bfloat162float(hi));
}

// feed-forward unit on the stacked [gate | up] product.  mode 0: g = min(gate, L), u = clamp(up, -L, L), y = g sigmoid(1.702 g) (u + 1);
// mode 1: y = silu(gate) up; mode 2: y = gelu(gate) up, gelu(z) = z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
// (ld: row stride of gu, 2 * ff when the product holds nothing else)
template <typename AT>
__global__ void k_seq_ff_act(AT* out, const float* gu, int ff, int N, float limit, int mode, int ld) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= (size_t)N * ff) return;
	const size_t n = i / ff, c = i % ff;
	if (mode == 1) {
		const float g = gu[n * ld + c];
		out[i] = to_act<AT>(g * sigmoidf_(g) * gu[n * ld + ff + c]);
		return;
	}
	if (mode == 2) {
		const float g = gu[n * ld + c];
		out[i] = to_act<AT>(0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * gu[n * ld + ff + c]);
		return;
	}
	const float g = fminf(gu[n * ld + c], limit);
	const float u = fminf(fmaxf(gu[n * ld + ff + c], -limit), limit);
	out[i] = to_act<AT>(g * sigmoidf_(1.702f * g) * (u + 1.f));
}

// y = silu(gate) up on TWO stacked products in one launch (the routed experts' rows and the shared unit's rows of one feed-forward)
struct FfPair {
	const float* gu[2];
	void* out[2];
	int ff[2], rows[2], ld[2];
};
template <typename AT>
__global__ void k_seq_ff_act2(FfPair a) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	const size_t n0 = (size_t)a.rows[0] * a.ff[0];
	const int k = i < n0 ? 0 : 1;
	if (k) i -= n0;
	if (i >= (size_t)a.rows[k] * a.ff[k]) return;
	const size_t n = i / a.ff[k], c = i % a.ff[k];
	const float g = a.gu[k][n * a.ld[k] + c];
	((AT*)a.out[k])[i] = to_act<AT>(g * sigmoidf_(g) * a.gu[k][n * a.ld[k] + a.ff[k] + c]);
}

// ---------------------------------------------------------------- short convolution + activation + per-head norm (+ cache append)

// One of q / k / v: `heads` vectors of `hd` channels starting at column `col` of the projection.
struct ConvSeg {
	int col, heads, hd;
	int act;     // 1: SiLU after the convolution
	int norm;    // 0 none, 1 unit vector (sum of squares + 1e-6), 2 RMS (mean of squares + eps)
	float mul;   // factor after the norm
	int to_cache;
	float* dst;  // [N][heads*hd], or the cache [rows][heads*hd]
};
struct ConvArgs {
	ConvSeg seg[3];
	const float* proj;
	int ldp;
	const bf16* w;      // [channels][taps]
	const bf16* bias = nullptr; // [channels] added after the taps, or null
	int pcol = 0;       // column of channel 0 in the projection (segment columns, weights and state count channels from 0)
	int taps, channels; // channels = all of q|k|v
	const float* state; // [slots][taps-1][channels]: the projected values of the taps-1 positions before the step
	float eps;
};
// one warp per (token, head vector)
__global__ void k_seq_conv_heads(ConvArgs a, SeqBatch sb) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int n = blockIdx.x;
	int u = blockIdx.y * (blockDim.x >> 5) + warp, s = 0;
	while (s < 3 && u >= a.seg[s].heads) u -= a.seg[s].heads, ++s;
	if (s == 3) return;
	const ConvSeg sg = a.seg[s];
	const int slot = sb.tslot[n], pos = sb.tpos[n];
	const int back = n - sb.tfirst[n]; // tokens of this step before this one
	const int T1 = a.taps - 1;
	const float* st = a.state + (size_t)slot * T1 * a.channels;
	float* d = sg.dst + (sg.to_cache ? cache_row(sb, slot, pos) : (long)n) * (sg.heads * sg.hd) + u * sg.hd;
	float ss = 0.f;
	for (int i = lane; i < sg.hd; i += 32) {
		const int ch = sg.col + u * sg.hd + i;
		float y = 0.f;
		for (int j = 0; j < a.taps; ++j) {
			const int ago = T1 - j; // tap j multiplies the value `ago` positions back
			const float v = ago <= back ? a.proj[(size_t)(n - ago) * a.ldp + a.pcol + ch] : st[(size_t)(T1 - (ago - back)) * a.channels + ch];
			y += ldf(a.w + (size_t)ch * a.taps + j) * v;
		}
		if (a.bias) y += ldf(a.bias + ch);
		if (sg.act) y = y * sigmoidf_(y);
		d[i] = y;
		ss += y * y;
	}
	if (sg.norm) {
		ss = warp_sum(ss);
		const float r = (sg.norm == 1 ? 1.f / sqrtf(ss + 1e-6f) : 1.f / sqrtf(ss / (float)sg.hd + a.eps)) * sg.mul;
		for (int i = lane; i < sg.hd; i += 32) d[i] *= r;
	}
}
// after the convolution: the state becomes the last taps-1 projected values of each sequence
__global__ void k_seq_conv_state(float* state, const float* proj, int ldp, int taps, int channels, SeqBatch sb, int pcol) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const int b = blockIdx.y, ch = blockIdx.x * blockDim.x + threadIdx.x;
	if (ch >= channels) return;
	const int T1 = taps - 1, cnt = sb.scount[b], start = sb.sstart[b];
	float* st = state + (size_t)sb.sslot[b] * T1 * channels;
	for (int i = 0; i < T1; ++i) { // new[i] = value T1 - i positions before the end; ascending i only reads old[i + cnt] with cnt >= 1
		const int ago = T1 - i;
		st[(size_t)i * channels + ch] = ago <= cnt ? proj[(size_t)(start + cnt - ago) * ldp + pcol + ch] : st[(size_t)(i + cnt) * channels + ch];
	}
}

// ---------------------------------------------------------------- attention over the paged cache
// One CTA per (token, tile of query heads that share one key/value head).  Keys: `kd` floats at column kcol of the K cache
// rows, values: `vd` floats at column vcol of the V cache rows (latent attention: both are the cached latent).  Softmax in
// fp32, online over chunks of ATT_KC keys; `sink` joins the denominator only; `gate` (raw, per token and head) multiplies
// the output through a sigmoid.
#define ATT_KC 64
#define ATT_THREADS 256
#define ATT_MAXI 32 // output elements per thread: heads of the tile x value columns per thread
#define ATT_KPL 16  // key channels per lane held in registers (keys up to 512 wide)
struct AttArgs {
	const float* q;   // [N][heads][kd]
	const float* kc;  // cache rows of width kld
	const float* vc;
	int kld, vld;
	int heads, group; // query heads per key/value head
	int tile;         // query heads per CTA (divides group)
	int kd, vd;
	int window;       // <= 0: all earlier positions
	int keep_first;   // with a window: positions below this stay visible to every later query
	int chunk = 0;    // > 0: only keys from floor(position / chunk) * chunk on are visible
	const float* slopes = nullptr; // [heads] or null: score -= slopes[h] * (query position - key position)
	int add_one = 0;  // 1: a sink of score zero (one added to the denominator); `sink` is then unused
	float scale;
	const bf16* sink; // [heads] or null
	const float* gate;
	int ldg, ghs, ges; // gate[n * ldg + h * ghs + d * ges]: one value per head (ghs 1, ges 0) or per output channel (ghs vd, ges 1)
	const int* skip;  // [N] or null: 1 = this token's attention is computed by the product path (k_seq_attn_*), the CTA leaves
	int nsplit;       // CTAs that share one (token, head tile)'s keys; > 1: partial results go to `part`, k_seq_attention_merge finishes
	float* part;      // [N][heads][nsplit][vd + 2]: unnormalised output, running maximum, denominator
	int split = 0;    // 1: on the product path queries, keys and probabilities travel as bf16 pairs (value + remainder), so scores and weights keep fp32 accuracy
};
template <typename AT>
__global__ void __launch_bounds__(ATT_THREADS) k_seq_attention(AttArgs a, AT* out, SeqBatch sb) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	extern __shared__ float sm[];
	const int n = blockIdx.x, h0 = blockIdx.y * a.tile, R = a.tile;
	if (a.skip && a.skip[n]) return;
	const int kvh = h0 / a.group;
	float* qs = sm;                  // [R][kd]
	float* sc = qs + ((R * a.kd + 3) & ~3); // [R][ATT_KC], 16-byte aligned
	float* mrow = sc + R * ATT_KC;   // [R] running maximum
	float* lrow = mrow + R;          // [R] running denominator
	float* frow = lrow + R;          // [R] rescale factor of this chunk
	__shared__ long rows[ATT_KC];    // cache rows of this chunk's keys
	__shared__ int dist[ATT_KC];     // distance of each key of the chunk from the query
	const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarp = ATT_THREADS / 32;
	const int slot = sb.tslot[n], pos = sb.tpos[n];
	int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
	if (a.chunk > 0) lo = max(lo, pos / a.chunk * a.chunk);
	// visible keys in order: the kept first positions the window has left behind, [0, kf), then the window [lo, pos]
	const int kf = min(a.keep_first, lo), total = kf + pos - lo + 1;
	// this CTA's share of the key chunks (the whole range when nsplit == 1)
	const int nchunk = (total + ATT_KC - 1) / ATT_KC, per = (nchunk + a.nsplit - 1) / a.nsplit;
	const int c_begin = (int)blockIdx.z * per * ATT_KC, c_end = min(total - 1, ((int)blockIdx.z + 1) * per * ATT_KC - 1);
	for (int i = tid; i < R * a.kd; i += ATT_THREADS) qs[i] = a.q[((size_t)n * a.heads + h0) * a.kd + i];
	if (tid < R) {
		const bool sk = (a.sink || a.add_one) && blockIdx.z == 0; // the sink counts once: in the first share
		mrow[tid] = sk ? (a.add_one ? 0.f : ldf(a.sink + h0 + tid)) : -INFINITY, lrow[tid] = sk ? 1.f : 0.f;
	}
	float acc[ATT_MAXI];
#pragma unroll
	for (int i = 0; i < ATT_MAXI; ++i) acc[i] = 0.f;
	const bool wide = a.vd > 2 * ATT_THREADS;
	__syncthreads();
	for (int c0 = c_begin; c0 <= c_end; c0 += ATT_KC) {
		const int nk = min(ATT_KC, total - c0);
		if (tid < ATT_KC) {
			const int kp = c0 + tid < kf ? c0 + tid : lo + c0 + tid - kf;
			rows[tid] = tid < nk ? cache_row(sb, slot, kp) : 0, dist[tid] = pos - kp;
		}
		__syncthreads();
		// scores: one warp per key, lanes across the key's channels; the lane's slice of the key is read once for all heads
		for (int j = warp; j < ATT_KC; j += nwarp) {
			if (j < nk) {
				const float* kr = a.kc + rows[j] * a.kld + (size_t)kvh * a.kd;
				if (a.kd <= 32 * ATT_KPL) {
					float kv[ATT_KPL];
#pragma unroll
					for (int i = 0; i < ATT_KPL; ++i) kv[i] = i * 32 + lane < a.kd ? kr[i * 32 + lane] : 0.f;
					for (int r0 = 0; r0 < R; r0 += 4) { // four heads' dot products advance together: independent chains and reductions
						float dd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
						for (int i = 0; i < ATT_KPL; ++i) {
							if (i * 32 < a.kd) {
								const float* qp = qs + r0 * a.kd + min(i * 32 + lane, a.kd - 1);
#pragma unroll
								for (int u = 0; u < 4; ++u)
									if (r0 + u < R) dd[u] = fmaf(qp[u * a.kd], kv[i], dd[u]);
							}
						}
#pragma unroll
						for (int u = 0; u < 4; ++u) dd[u] = warp_sum(dd[u]);
#pragma unroll
						for (int u = 0; u < 4; ++u)
							if (r0 + u < R && lane == u) sc[(r0 + u) * ATT_KC + j] = dd[u] * a.scale - (a.slopes ? a.slopes[h0 + r0 + u] * (float)dist[j] : 0.f);
					}
				} else {
					for (int r = 0; r < R; ++r) {
						float d = 0.f;
						for (int i = lane; i < a.kd; i += 32) d += qs[r * a.kd + i] * kr[i];
						d = warp_sum(d);
						if (lane == 0) sc[r * ATT_KC + j] = d * a.scale - (a.slopes ? a.slopes[h0 + r] * (float)dist[j] : 0.f);
					}
				}
			} else if (lane == 0) {
				for (int r = 0; r < R; ++r) sc[r * ATT_KC + j] = -INFINITY;
			}
		}
		__syncthreads();
		// running maximum, probabilities in place, denominator
		for (int r = warp; r < R; r += nwarp) {
			float mx = -INFINITY;
			for (int j = lane; j < ATT_KC; j += 32) mx = fmaxf(mx, sc[r * ATT_KC + j]);
			mx = warp_max(mx);
			const float mo = mrow[r], mn = fmaxf(mo, mx);
			float ps = 0.f;
			for (int j = lane; j < ATT_KC; j += 32) {
				const float p = expf(sc[r * ATT_KC + j] - mn);
				sc[r * ATT_KC + j] = p, ps += p;
			}
			ps = warp_sum(ps);
			if (lane == 0) {
				const float f = mo == -INFINITY ? 0.f : expf(mo - mn);
				frow[r] = f, lrow[r] = lrow[r] * f + ps, mrow[r] = mn;
			}
		}
		__syncthreads();
		// values: a thread owns value columns tid and tid + 256 for every head of the tile (accumulator c * 16 + r); values wider
		// than 512 run one head per CTA with up to 32 columns per thread (accumulator c)
		if (wide) {
#pragma unroll
			for (int k = 0; k < ATT_MAXI; ++k) {
				const int d = tid + k * ATT_THREADS;
				if (d < a.vd) {
					const float* vcol = a.vc + (size_t)kvh * a.vd + d;
					float s = acc[k] * frow[0];
					for (int j = 0; j < nk; ++j) s = fmaf(sc[j], vcol[rows[j] * a.vld], s);
					acc[k] = s;
				}
			}
		} else {
#pragma unroll
			for (int c = 0; c < 2; ++c) {
				const int d = tid + c * ATT_THREADS;
				if (d < a.vd) {
					const float* vcol = a.vc + (size_t)kvh * a.vd + d;
#pragma unroll
					for (int r = 0; r < 16; ++r)
						if (r < R) acc[c * 16 + r] *= frow[r];
					for (int j0 = 0; j0 < nk; j0 += 4) {
						float v[4];
#pragma unroll
						for (int u = 0; u < 4; ++u) v[u] = j0 + u < nk ? vcol[rows[j0 + u] * a.vld] : 0.f;
#pragma unroll
						for (int r = 0; r < 16; ++r) {
							if (r < R) {
								const float4 p = *(const float4*)(sc + r * ATT_KC + j0);
								acc[c * 16 + r] = fmaf(p.w, v[3], fmaf(p.z, v[2], fmaf(p.y, v[1], fmaf(p.x, v[0], acc[c * 16 + r]))));
							}
						}
					}
				}
			}
		}
		__syncthreads();
	}
	// accumulator k -> (head of the tile, value column)
	auto head_of = [&](int k) { return wide ? 0 : k % 16; };
	auto col_of = [&](int k) { return tid + (wide ? k : k / 16) * ATT_THREADS; };
	if (a.nsplit > 1) {
		const int pw = a.vd + 2;
#pragma unroll
		for (int k = 0; k < ATT_MAXI; ++k) {
			const int r = head_of(k), d = col_of(k);
			if (r < R && d < a.vd) a.part[(((size_t)n * a.heads + h0 + r) * a.nsplit + blockIdx.z) * pw + d] = acc[k];
		}
		if (tid < R) {
			float* p = a.part + (((size_t)n * a.heads + h0 + tid) * a.nsplit + blockIdx.z) * pw + a.vd;
			p[0] = mrow[tid], p[1] = lrow[tid];
		}
		return;
	}
#pragma unroll
	for (int k = 0; k < ATT_MAXI; ++k) {
		const int r = head_of(k), d = col_of(k);
		if (r < R && d < a.vd) {
			float v = acc[k] / lrow[r];
			if (a.gate) v *= sigmoidf_(a.gate[(size_t)n * a.ldg + (size_t)(h0 + r) * a.ghs + (size_t)d * a.ges]);
			out[((size_t)n * a.heads + h0 + r) * a.vd + d] = to_act<AT>(v);
		}
	}
}
// folds the shares of one (token, head) in share order: one CTA per (token, head)
template <typename AT>
__global__ void k_seq_attention_merge(AttArgs a, AT* out) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const int n = blockIdx.x, h = blockIdx.y, pw = a.vd + 2;
	if (a.skip && a.skip[n]) return;
	const float* p = a.part + ((size_t)n * a.heads + h) * a.nsplit * pw;
	float mx = -INFINITY;
	for (int z = 0; z < a.nsplit; ++z) mx = fmaxf(mx, p[z * pw + a.vd]);
	float l = 0.f;
	for (int z = 0; z < a.nsplit; ++z) {
		const float m = p[z * pw + a.vd];
		if (m != -INFINITY) l += p[z * pw + a.vd + 1] * expf(m - mx);
	}
	for (int d = threadIdx.x; d < a.vd; d += blockDim.x) {
		const float g = (a.gate ? sigmoidf_(a.gate[(size_t)n * a.ldg + (size_t)h * a.ghs + (size_t)d * a.ges]) : 1.f) / l;
		float v = 0.f;
		for (int z = 0; z < a.nsplit; ++z) {
			const float m = p[z * pw + a.vd];
			if (m != -INFINITY) v += p[z * pw + d] * expf(m - mx);
		}
		out[((size_t)n * a.heads + h) * a.vd + d] = to_act<AT>(v * g);
	}
}

// ---------------------------------------------------------------- prompt attention as products
// For many query tokens of one sequence the scores and the weighted values are matrix products on the tensor cores:
// the keys of the visible range are gathered from the paged cache into a bf16 matrix (values transposed), S = Q K^T per
// head, a row-wise fp32 softmax applies scale, causal / window mask, sink and output gate and writes bf16 probabilities,
// then O = P V.  k_seq_attention above serves single decoded tokens, short portions and the exact mode.
struct AttGather {
	const float* kc;
	const float* vc;
	int kld, vld, kcol, vcol; // column of this key/value head inside a cache row
	int kd, vd;
	bf16* Kb;   // [C][kd]
	bf16* Vt;   // [vd][Cp]
	int slot, k0, C, Cp;
	int kfb;    // the first kfb gathered keys are positions 0 .. kfb-1 (kept first tokens), the rest k0, k0 + 1, ...
	int split;  // 1: Kb rows are [hi | lo | hi] (3 kd wide: a key as a bf16 value and the bf16 of what the rounding left), Vt rows hold the values twice ([vd][2 Cp])
};
__global__ void k_seq_attn_gather(AttGather a, SeqBatch sb) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	__shared__ float tile[32][33];
	const int j0 = blockIdx.x * 32, tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8 threads
	const int dmax = max(a.kd, a.vd);
	for (int d0 = blockIdx.y * 32; d0 < dmax; d0 += gridDim.y * 32) {
		for (int r = ty; r < 32; r += 8) {
			const int j = j0 + r, d = d0 + tx;
			if (j < a.C) {
				const long row = cache_row(sb, a.slot, j < a.kfb ? j : a.k0 + j - a.kfb);
				if (d < a.kd) {
					const float kv = a.kc[row * a.kld + a.kcol + d];
					const bf16 hi = __float2bfloat16_rn(kv);
					if (a.split) {
						bf16* kr = a.Kb + (size_t)j * 3 * a.kd;
						kr[d] = hi, kr[a.kd + d] = __float2bfloat16_rn(kv - __bfloat162float(hi)), kr[2 * a.kd + d] = hi;
					} else a.Kb[(size_t)j * a.kd + d] = hi;
				}
				tile[r][tx] = d < a.vd ? a.vc[row * a.vld + a.vcol + d] : 0.f;
			} else tile[r][tx] = 0.f;
		}
		__syncthreads();
		for (int r = ty; r < 32; r += 8) {
			const int d = d0 + r, j = j0 + tx;
			if (d < a.vd && j < a.Cp) {
				const bf16 v = __float2bfloat16_rn(tile[tx][r]);
				if (a.split) a.Vt[(size_t)d * 2 * a.Cp + j] = v, a.Vt[(size_t)d * 2 * a.Cp + a.Cp + j] = v;
				else a.Vt[(size_t)d * a.Cp + j] = v;
			}
		}
		__syncthreads();
	}
}
struct AttSoftmax {
	const float* S; // [heads of the launch][T][Cp]
	bf16* P;        // same shape
	int T, C, Cp;
	int qpos0, k0, window;
	int chunk = 0;       // > 0: a row sees only positions from floor(position / chunk) * chunk on
	const float* slopes = nullptr; // already offset to the first head of the launch, or null: score -= slopes[z] * (row position - column position)
	int add_one = 0;     // 1: one added to the denominator
	int keep_first, kfb; // columns below kfb are the kept first positions 0 .. kfb-1; column j >= kfb is position k0 + j - kfb
	float scale;
	const bf16* sink; // already offset to the first head of the launch, or null
	const float* gate; // per head: gate[t * ldg + z], already offset to the first token and head, or null (per-channel gates are applied by the caller)
	int ldg;
	int split = 0;     // 1: P rows are 2 Cp wide: the probabilities as bf16, then the bf16 of what that rounding left
};
__global__ void __launch_bounds__(256) k_seq_attn_softmax(AttSoftmax a) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	__shared__ float red[8];
	__shared__ float bc;
	const int t = blockIdx.x, z = blockIdx.y, tid = threadIdx.x;
	const float* srow = a.S + ((size_t)z * a.T + t) * a.Cp;
	bf16* prow = a.P + ((size_t)z * a.T + t) * a.Cp * (a.split ? 2 : 1);
	const int qpos = a.qpos0 + t;
	const int hi = min(a.C - 1, qpos - a.k0 + a.kfb); // last visible column
	int wlo = a.window > 0 ? qpos - a.window + 1 : 0;
	if (a.chunk > 0) wlo = max(wlo, qpos / a.chunk * a.chunk);
	const int lo = a.kfb > 0 || a.keep_first > a.k0 ? 0 : max(0, wlo - a.k0); // nothing is visible before this column
	auto seen = [&](int j) { // column j's position: a kept first token, or inside the window (j <= hi is the causal bound)
		const int p = j < a.kfb ? j : a.k0 + j - a.kfb;
		return p >= wlo || p < a.keep_first;
	};
	const float sk = a.add_one ? 0.f : a.sink ? ldf(a.sink + z) : -INFINITY;
	const float slope = a.slopes ? a.slopes[z] : 0.f;
	auto score = [&](int j) { return srow[j] * a.scale - slope * (float)(qpos - (j < a.kfb ? j : a.k0 + j - a.kfb)); };
	float mx = sk;
	for (int j = lo + tid; j <= hi; j += 256)
		if (seen(j)) mx = fmaxf(mx, score(j));
	mx = warp_max(mx);
	if ((tid & 31) == 0) red[tid >> 5] = mx;
	__syncthreads();
	if (tid == 0) {
		for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
		bc = mx;
	}
	__syncthreads();
	mx = bc;
	float sum = 0.f;
	for (int j = lo + tid; j <= hi; j += 256)
		if (seen(j)) sum += expf(score(j) - mx);
	sum = warp_sum(sum);
	__syncthreads();
	if ((tid & 31) == 0) red[tid >> 5] = sum;
	__syncthreads();
	if (tid == 0) {
		for (int w = 1; w < 8; ++w) sum += red[w];
		if (a.sink || a.add_one) sum += expf(sk - mx);
		bc = (a.gate ? sigmoidf_(a.gate[(size_t)t * a.ldg + z]) : 1.f) / sum;
	}
	__syncthreads();
	const float f = bc;
	for (int j = tid; j < a.Cp; j += 256) {
		const float p = j >= lo && j <= hi && seen(j) ? expf(score(j) - mx) * f : 0.f;
		const bf16 ph = __float2bfloat16_rn(p);
		prow[j] = ph;
		if (a.split) prow[a.Cp + j] = __float2bfloat16_rn(p - __bfloat162float(ph));
	}
}

// ---------------------------------------------------------------- gated delta rule
// One CTA per (sequence, head): the head's state S [dim][vdim] sits in shared memory for all tokens of the step, thread j
// owns value column j.  Per token:  S <- g (.) S (rows);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
// g = exp(-exp(A_log) softplus(dt + dt_bias)) and beta = sigmoid(.) are formed here in fp32.
struct DeltaArgs {
	const float *q, *k, *v; // [N][kv_heads*dim] x2, [N][heads*vdim]
	const float* proj;      // beta (raw) at column bcol
	int ldp, bcol;
	const float* dt;        // [N][heads*dim] raw
	const bf16 *a_log, *dt_bias;
	float* state;           // [slots][heads][dim][vdim]
	float* o;               // [N][heads*vdim]
	int heads, kv_heads, dim, vdim;
};
__global__ void k_seq_delta_scan(DeltaArgs a, SeqBatch sb) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	extern __shared__ float sm[];
	const int b = blockIdx.x, h = blockIdx.y, D = a.dim, V = a.vdim;
	const int kh = h / (a.heads / a.kv_heads);
	float* S = sm;          // [D][V]
	float* ks = S + D * V;  // [D]
	float* qs = ks + D;
	float* gs = qs + D;
	const int tid = threadIdx.x;
	float* Sg = a.state + ((size_t)sb.sslot[b] * a.heads + h) * D * V;
	for (int i = tid; i < D * V; i += blockDim.x) S[i] = Sg[i];
	const float A = expf(ldf(a.a_log + h));
	const int start = sb.sstart[b], cnt = sb.scount[b];
	for (int t = 0; t < cnt; ++t) {
		const int n = start + t;
		__syncthreads();
		for (int i = tid; i < D; i += blockDim.x) {
			ks[i] = a.k[((size_t)n * a.kv_heads + kh) * D + i];
			qs[i] = a.q[((size_t)n * a.kv_heads + kh) * D + i];
			gs[i] = expf(-A * softplusf_(a.dt[((size_t)n * a.heads + h) * D + i] + ldf(a.dt_bias + h * D + i)));
		}
		__syncthreads();
		if (tid < V) {
			float dot = 0.f;
			for (int i = 0; i < D; ++i) {
				const float s = gs[i] * S[i * V + tid];
				S[i * V + tid] = s;
				dot += s * ks[i];
			}
			const float beta = sigmoidf_(a.proj[(size_t)n * a.ldp + a.bcol + h]);
			const float u = beta * (a.v[((size_t)n * a.heads + h) * V + tid] - dot);
			float o = 0.f;
			for (int i = 0; i < D; ++i) {
				const float s = S[i * V + tid] + ks[i] * u;
				S[i * V + tid] = s;
				o += s * qs[i];
			}
			a.o[((size_t)n * a.heads + h) * V + tid] = o;
		}
	}
	__syncthreads();
	for (int i = tid; i < D * V; i += blockDim.x) Sg[i] = S[i];
}
// The same recurrence with the state in registers: four lanes share a value column, each holding D/4 of its rows.  Tokens are
// staged DELTA_TB at a time: while one block of tokens is applied (no barrier between its tokens, only shuffles inside a
// column's four lanes), the next block's k, q, decay, v and beta travel from global memory into the other half of a double
// buffer; k, q and the decay are read back as float4 (quarters padded by 4 floats: the four lanes hit different banks).
#define DELTA_TB 4
template <int D>
__global__ void __launch_bounds__(512) k_seq_delta_scan_reg(DeltaArgs a, SeqBatch sb) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	constexpr int Q = D / 4, QP = Q + 4;
	extern __shared__ __align__(16) float sm[];
	const int b = blockIdx.x, h = blockIdx.y, V = a.vdim;
	const int kh = h / (a.heads / a.kv_heads);
	const int tid = threadIdx.x, part = tid & 3;
	const bool live = (tid >> 2) < V;          // lanes past the last column run along on a copy of it (whole warps shuffle)
	const int col = live ? tid >> 2 : V - 1;
	const int vpad = (V + 1 + 3) & ~3;         // v and beta of a token, rounded so that the next token stays 16-byte aligned
	const int tok_len = 3 * 4 * QP + vpad;     // k, q, g (padded quarters), v, beta
	float* buf[2] = {sm, sm + DELTA_TB * tok_len};
	float S[Q];
	float* Sg = a.state + ((size_t)sb.sslot[b] * a.heads + h) * D * V;
#pragma unroll
	for (int i = 0; i < Q; ++i) S[i] = Sg[(size_t)(part * Q + i) * V + col];
	const float A = expf(ldf(a.a_log + h));
	const int start = sb.sstart[b], cnt = sb.scount[b];
	// Staging.  A token's inputs are 3 D / 4 + V / 4 float4 items (k, q, raw decay input, v) and one scalar (beta's input); item e of a
	// block belongs to token e / items4.  Thread tid serves items tid and tid + blockDim of every block, so where an item comes from
	// and where it goes is worked out once; per block a thread issues its (at most two) 16-byte loads before the running block's
	// arithmetic and finishes them (decay, beta) into the other buffer after it.
	const int items4 = (3 * D + V) / 4 + 1;
	const float* src[2];
	const bf16* biasp[2];            // decay items: their four dt_bias entries
	int stride[2], slot[2], kind[2]; // kind: 0 plain float4, 1 decay input, 2 beta input (scalar), -1 none
#pragma unroll
	for (int r = 0; r < 2; ++r) {
		const int e = tid + r * (int)blockDim.x, tt = e / items4, it4 = e % items4;
		kind[r] = -1, src[r] = a.k, stride[r] = 0, slot[r] = 0, biasp[r] = a.dt_bias;
		if (tt < DELTA_TB) {
			const int i0 = 4 * it4;
			if (i0 < 3 * D) {
				const int seg = i0 / D, w = i0 % D;
				kind[r] = seg == 2 ? 1 : 0;
				biasp[r] = a.dt_bias + h * D + w;
				stride[r] = seg == 2 ? a.heads * D : a.kv_heads * D;
				src[r] = (seg == 0 ? a.k + (size_t)kh * D : seg == 1 ? a.q + (size_t)kh * D : a.dt + (size_t)h * D) + w + (size_t)(start + tt) * stride[r];
				slot[r] = tt * tok_len + seg * 4 * QP + (w / Q) * QP + w % Q;
			} else if (i0 < 3 * D + V) {
				kind[r] = 0, stride[r] = a.heads * V;
				src[r] = a.v + (size_t)h * V + (i0 - 3 * D) + (size_t)(start + tt) * stride[r];
				slot[r] = tt * tok_len + 3 * 4 * QP + i0 - 3 * D;
			} else {
				kind[r] = 2, stride[r] = a.ldp;
				src[r] = a.proj + a.bcol + h + (size_t)(start + tt) * stride[r];
				slot[r] = tt * tok_len + 3 * 4 * QP + V;
			}
		}
	}
	const int tt_of[2] = {tid / items4, (tid + (int)blockDim.x) / items4};
	auto fetch_block = [&](int blk, float4 (&pre)[2]) {
		const int nt = min(DELTA_TB, cnt - blk * DELTA_TB);
#pragma unroll
		for (int r = 0; r < 2; ++r) {
			pre[r] = make_float4(0.f, 0.f, 0.f, 0.f);
			if (kind[r] >= 0 && tt_of[r] < nt) {
				const float* p = src[r] + (size_t)blk * DELTA_TB * stride[r];
				if (kind[r] == 2) pre[r].x = __ldg(p);
				else pre[r] = __ldg((const float4*)p);
			}
		}
	};
	auto put_block = [&](float* st, int blk, const float4 (&pre)[2]) {
		const int nt = min(DELTA_TB, cnt - blk * DELTA_TB);
#pragma unroll
		for (int r = 0; r < 2; ++r) {
			if (kind[r] >= 0 && tt_of[r] < nt) {
				float4 v = pre[r];
				if (kind[r] == 1) {
					const bf16* bias = biasp[r];
					v.x = expf(-A * softplusf_(v.x + ldf(bias))), v.y = expf(-A * softplusf_(v.y + ldf(bias + 1)));
					v.z = expf(-A * softplusf_(v.z + ldf(bias + 2))), v.w = expf(-A * softplusf_(v.w + ldf(bias + 3)));
				}
				if (kind[r] == 2) st[slot[r]] = sigmoidf_(v.x);
				else *(float4*)(st + slot[r]) = v;
			}
		}
	};
	const int nblk = (cnt + DELTA_TB - 1) / DELTA_TB;
	float4 pre[2];
	fetch_block(0, pre);
	put_block(buf[0], 0, pre);
	__syncthreads();
	for (int blk = 0; blk < nblk; ++blk) {
		const float* cur = buf[blk & 1];
		if (blk + 1 < nblk) fetch_block(blk + 1, pre);
		const int nt = min(DELTA_TB, cnt - blk * DELTA_TB);
		for (int tt = 0; tt < nt; ++tt) {
			const float* tk = cur + tt * tok_len;
			const float4 *ks = (const float4*)(tk + part * QP), *qs = (const float4*)(tk + 4 * QP + part * QP), *gs = (const float4*)(tk + 8 * QP + part * QP);
			float dot = 0.f;
#pragma unroll
			for (int i = 0; i < Q / 4; ++i) {
				const float4 g4 = gs[i], k4 = ks[i];
				S[4 * i] *= g4.x, S[4 * i + 1] *= g4.y, S[4 * i + 2] *= g4.z, S[4 * i + 3] *= g4.w;
				dot = fmaf(S[4 * i], k4.x, dot), dot = fmaf(S[4 * i + 1], k4.y, dot), dot = fmaf(S[4 * i + 2], k4.z, dot), dot = fmaf(S[4 * i + 3], k4.w, dot);
			}
			dot += __shfl_xor_sync(0xffffffffu, dot, 1);
			dot += __shfl_xor_sync(0xffffffffu, dot, 2);
			const float u = tk[3 * 4 * QP + V] * (tk[3 * 4 * QP + col] - dot);
			float o = 0.f;
#pragma unroll
			for (int i = 0; i < Q / 4; ++i) {
				const float4 k4 = ks[i], q4 = qs[i];
				S[4 * i] = fmaf(k4.x, u, S[4 * i]), S[4 * i + 1] = fmaf(k4.y, u, S[4 * i + 1]), S[4 * i + 2] = fmaf(k4.z, u, S[4 * i + 2]), S[4 * i + 3] = fmaf(k4.w, u, S[4 * i + 3]);
				o = fmaf(S[4 * i], q4.x, o), o = fmaf(S[4 * i + 1], q4.y, o), o = fmaf(S[4 * i + 2], q4.z, o), o = fmaf(S[4 * i + 3], q4.w, o);
			}
			o += __shfl_xor_sync(0xffffffffu, o, 1);
			o += __shfl_xor_sync(0xffffffffu, o, 2);
			if (part == 0 && live) a.o[((size_t)(start + blk * DELTA_TB + tt) * a.heads + h) * V + col] = o;
		}
		if (blk + 1 < nblk) put_block(buf[(blk + 1) & 1], blk + 1, pre);
		__syncthreads();
	}
	if (live) {
#pragma unroll
		for (int i = 0; i < Q; ++i) Sg[(size_t)(part * Q + i) * V + col] = S[i];
	}
}
// read-out: o / rms(o) (per head) * w * sigmoid(gate); one warp per (token, head)
// (the gate goes through a sigmoid, or through SiLU when silu_gate is set; it is read at gate[token * ldg + head * vdim + i])
template <typename AT>
__global__ void k_seq_delta_out(AT* out, const float* o, const float* gate, int ldg, const bf16* w, int N, int heads, int vdim, float eps, int silu_gate) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const size_t u = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
	if (u >= (size_t)N * heads) return;
	const float* src = o + u * vdim;
	float ss = 0.f;
	for (int i = lane; i < vdim; i += 32) ss += src[i] * src[i];
	ss = warp_sum(ss);
	const float r = 1.f / sqrtf(ss / (float)vdim + eps);
	const float* gp = gate + (u / heads) * (size_t)ldg + (u % heads) * (size_t)vdim;
	for (int i = lane; i < vdim; i += 32) {
		const float g = gp[i], sg = sigmoidf_(g);
		out[u * vdim + i] = to_act<AT>(src[i] * r * ldf(w + i) * (silu_gate ? g * sg : sg));
	}
}

// ---------------------------------------------------------------- gated linear attention
// Per (sequence, head): S [dim][vdim] fp32;  per token  S <- diag(a) S + k v^T,  o = S^T q * qscale  with one decay a per key
// channel (formed in fp32 by the decay projection's epilogue, EPI_DECAY).  q, k, v are columns of the stacked projection (row
// stride ldp).
struct GlaArgs {
	const float* proj;
	int ldp, qcol, kcol, vcol;
	const float* decay;  // [N][heads*dim]
	float qscale;
	float* state;        // [slots][heads][vdim][ldstate]: a value column's key channels side by side (channels past dim stay zero)
	int ldstate;
	float* o;            // [N][heads*vdim]
	int heads, dim, vdim;
	int vec;             // rows, columns and bases are 16-byte aligned: tokens are staged with 16-byte copies instead of 4-byte ones
};
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
	asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// One CTA of 128 threads per (sequence, head, 128 / P value columns).  The state sits in registers: P lanes share a value column,
// each holding R of its key channels (P = 4, 8 or 16: the host takes more lanes per column when sequences x heads alone would
// leave SMs idle, since per token a warp issues ~3 R arithmetic instructions and that, not memory, bounds a long prompt).
// Tokens are staged GLA_TB at a time into a double buffer with asynchronous copies (k, q and the decay in P segments padded by 4
// floats, so that the lanes of a column read different banks as float4; the CTA's values of v), so a block's tokens are applied
// without a barrier between them -- log2(P) shuffles fold a column's read-out -- while the next block travels.  Read-outs
// leave through shared memory, one coalesced store per block.
#define GLA_TB 16
template <int R, int P>
__global__ void __launch_bounds__(128) k_seq_gla_scan(GlaArgs a, SeqBatch sb) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	constexpr int QP = R + 4, VC = 128 / P, TOK = 3 * P * QP + VC;
	extern __shared__ __align__(16) float sm[];
	float* const buf0 = sm;
	float* const obuf = sm + 2 * GLA_TB * TOK; // [2][GLA_TB][VC]
	const int b = blockIdx.x, h = blockIdx.y, D = a.dim, V = a.vdim, v0 = blockIdx.z * VC;
	const int tid = threadIdx.x, part = tid % P, cl = tid / P;
	const bool live = v0 + cl < V;
	const int start = sb.sstart[b], cnt = sb.scount[b], nblk = (cnt + GLA_TB - 1) / GLA_TB;
	// the padding (channels past dim, columns past vdim) is never copied over: zero what this step will use, once
	for (int i = tid; i < min(cnt, 2 * GLA_TB) * TOK; i += 128) sm[i] = 0.f;
	float S[R];
	float* Sg = a.state + (((size_t)sb.sslot[b] * a.heads + h) * V + min(v0 + cl, V - 1)) * a.ldstate + part * R;
#pragma unroll
	for (int i = 0; i < R; i += 4) {
		const float4 t = *(const float4*)(Sg + i);
		S[i] = t.x, S[i + 1] = t.y, S[i + 2] = t.z, S[i + 3] = t.w;
	}
	// 16-byte staging: a thread copies the same (at most two) chunks of every token, so where they come from and go to is worked out once
	const float* vsrc[2] = {nullptr, nullptr};
	long vstride[2] = {0, 0};
	int vdst[2] = {0, 0};
	if (a.vec) {
		const int dc = D / 4;
#pragma unroll
		for (int r = 0; r < 2; ++r) {
			const int c = tid + r * 128;
			if (c < 3 * dc) {
				const int sgm = c / dc, i = 4 * (c % dc);
				vsrc[r] = sgm == 2 ? a.decay + ((size_t)start * a.heads + h) * D + i : a.proj + (size_t)start * a.ldp + (sgm == 0 ? a.kcol : a.qcol) + h * D + i;
				vstride[r] = sgm == 2 ? (long)a.heads * D : a.ldp;
				vdst[r] = sgm * P * QP + (i / R) * QP + i % R;
			} else if (c < 3 * dc + VC / 4 && v0 + 4 * (c - 3 * dc) < V) {
				const int i = 4 * (c - 3 * dc);
				vsrc[r] = a.proj + (size_t)start * a.ldp + a.vcol + h * V + v0 + i, vstride[r] = a.ldp, vdst[r] = 3 * P * QP + i;
			}
		}
	}
	__syncthreads();
	auto issue = [&](int blk) {
		float* dst = buf0 + (blk & 1) * GLA_TB * TOK;
		const int t0 = blk * GLA_TB, nt = min(GLA_TB, cnt - t0);
		if (a.vec) {
#pragma unroll
			for (int r = 0; r < 2; ++r)
				if (vsrc[r])
					for (int tt = 0; tt < nt; ++tt) cp_async16(dst + tt * TOK + vdst[r], vsrc[r] + (t0 + tt) * vstride[r]);
		} else {
			const int per = 3 * D + VC;
			for (int e = tid; e < nt * per; e += 128) {
				const int tt = e / per, c = e % per;
				const float* row = a.proj + (size_t)(start + t0 + tt) * a.ldp;
				if (c < 3 * D) {
					const int sgm = c / D, i = c % D;
					const float* src = sgm == 0 ? row + a.kcol + h * D + i : sgm == 1 ? row + a.qcol + h * D + i : a.decay + ((size_t)(start + t0 + tt) * a.heads + h) * D + i;
					cp_async4(dst + tt * TOK + sgm * P * QP + (i / R) * QP + i % R, src);
				} else {
					const int i = c - 3 * D;
					if (v0 + i < V) cp_async4(dst + tt * TOK + 3 * P * QP + i, row + a.vcol + h * V + v0 + i);
				}
			}
		}
		asm volatile("cp.async.commit_group;" ::: "memory");
	};
	auto write_out = [&](int blk) { // the read-outs of a finished block: consecutive threads, consecutive columns
		const int nt = min(GLA_TB, cnt - blk * GLA_TB);
		const float* ob = obuf + (blk & 1) * GLA_TB * VC;
		for (int e = tid; e < nt * VC; e += 128) {
			const int tt = e / VC, c = e % VC;
			if (v0 + c < V) a.o[((size_t)(start + blk * GLA_TB + tt) * a.heads + h) * V + v0 + c] = ob[e];
		}
	};
	issue(0);
	for (int blk = 0; blk < nblk; ++blk) {
		if (blk + 1 < nblk) {
			issue(blk + 1);
			asm volatile("cp.async.wait_group 1;" ::: "memory");
		} else {
			asm volatile("cp.async.wait_group 0;" ::: "memory");
		}
		__syncthreads();
		if (blk > 0) write_out(blk - 1);
		const float* __restrict__ cur = buf0 + (blk & 1) * GLA_TB * TOK;
		float* __restrict__ ob = obuf + (blk & 1) * GLA_TB * VC;
		const int nt = min(GLA_TB, cnt - blk * GLA_TB);
		// the block's tokens, unrolled: each lane's share of a read-out stays in a register until the block is done, then the shares are
		// folded for all tokens at once -- independent shuffles that overlap, instead of one dependent chain per token
		float oacc[GLA_TB];
		auto apply = [&](int tt) { // one token: decay, write, this lane's share of the read-out
			const float* tk = cur + tt * TOK;
			const float4 *kp = (const float4*)(tk + part * QP), *qp = (const float4*)(tk + P * QP + part * QP), *gp = (const float4*)(tk + 2 * P * QP + part * QP);
			const float v = tk[3 * P * QP + cl];
			float o0 = 0.f, o1 = 0.f;
#pragma unroll
			for (int i = 0; i < R / 4; ++i) {
				const float4 g4 = gp[i], k4 = kp[i], q4 = qp[i];
				S[4 * i] = fmaf(g4.x, S[4 * i], k4.x * v), S[4 * i + 1] = fmaf(g4.y, S[4 * i + 1], k4.y * v);
				S[4 * i + 2] = fmaf(g4.z, S[4 * i + 2], k4.z * v), S[4 * i + 3] = fmaf(g4.w, S[4 * i + 3], k4.w * v);
				o0 = fmaf(S[4 * i], q4.x, o0), o1 = fmaf(S[4 * i + 1], q4.y, o1), o0 = fmaf(S[4 * i + 2], q4.z, o0), o1 = fmaf(S[4 * i + 3], q4.w, o1);
			}
			return o0 + o1;
		};
		if (nt == GLA_TB) { // a full block has no branch between its tokens: the loads of later tokens move up past the arithmetic of earlier ones
#pragma unroll
			for (int tt = 0; tt < GLA_TB; ++tt) oacc[tt] = apply(tt);
		} else {
#pragma unroll
			for (int tt = 0; tt < GLA_TB; ++tt) oacc[tt] = tt < nt ? apply(tt) : 0.f;
		}
#pragma unroll
		for (int w = 1; w < P; w <<= 1)
#pragma unroll
			for (int tt = 0; tt < GLA_TB; ++tt) oacc[tt] += __shfl_xor_sync(0xffffffffu, oacc[tt], w);
#pragma unroll
		for (int tt = 0; tt < GLA_TB; ++tt)
			if (tt % P == part) ob[tt * VC + cl] = oacc[tt] * a.qscale; // every lane of a column holds the sums: the lanes share the stores out
		__syncthreads(); // this block's buffer may be refilled and its read-outs are complete
	}
	write_out(nblk - 1);
	if (live) {
#pragma unroll
		for (int i = 0; i < R; i += 4) *(float4*)(Sg + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
	}
}

// ---------------------------------------------------------------- query / key preparation of grouped-query attention
// One CTA per token, on the stacked (biased) projection [q | k | v | ...]: an RMS norm over the WHOLE query projection and one over
// the whole key projection (all heads at once, weights qw / kw; null: no norm), then the first rot_dims channels of every head turn
// by the token's position (channel i with channel i + rot_dims/2, angle = position * freq[i], cos and sin times `mag`); queries go
// to an activation-independent fp32 matrix, keys and values to their cache rows.  Angles are formed in double: a position in the
// thousands times a frequency near one leaves fp32 with too few fraction bits.
struct QkArgs {
	const float* proj;
	int ldp;
	int heads, kv_heads, dim, vdim;
	const bf16 *qw, *kw;
	float eps;
	int rot_dims;
	const double* freq; // [rot_dims / 2]
	float mag;
	float* q;           // [N][heads*dim]
	float* kc;          // cache rows [kv_heads*dim]
	float* vc;          // cache rows [kv_heads*vdim]
	int v_norm = 0;     // 1: every value head is divided by its root mean square over vdim (eps inside the root, no weight)
	int per_head = 0;   // 1: the RMS norms run over each head's `dim` channels, qw / kw are [dim] and serve every head
};
__global__ void __launch_bounds__(256) k_seq_qk_rope(QkArgs a, SeqBatch sb) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	extern __shared__ float cs[]; // [rot_dims/2] cos, [rot_dims/2] sin, then (per_head) [heads + kv_heads] reciprocal root mean squares
	__shared__ float red[2][8];
	const int n = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
	const int Q = a.heads * a.dim, K = a.kv_heads * a.dim, Vn = a.kv_heads * a.vdim, half = a.rot_dims / 2;
	const float* pr = a.proj + (size_t)n * a.ldp;
	const int pos = sb.tpos[n];
	const long row = cache_row(sb, sb.tslot[n], pos);
	for (int i = tid; i < half; i += blockDim.x) {
		double s, c;
		sincos((double)pos * a.freq[i], &s, &c);
		cs[i] = (float)c * a.mag, cs[half + i] = (float)s * a.mag;
	}
	float sq = 0.f, sk = 0.f;
	float* rh = cs + 2 * max(half, 1);
	if (a.qw && a.per_head) { // one warp per head vector, query heads first: the key heads follow them in the projection
		for (int u = warp; u < a.heads + a.kv_heads; u += (int)(blockDim.x >> 5)) {
			const float* src = pr + (size_t)u * a.dim;
			float ss = 0.f;
			for (int i = lane; i < a.dim; i += 32) ss = fmaf(src[i], src[i], ss);
			ss = warp_sum(ss);
			if (lane == 0) rh[u] = 1.f / sqrtf(ss / (float)a.dim + a.eps);
		}
	} else if (a.qw) {
		for (int i = tid; i < Q; i += blockDim.x) sq = fmaf(pr[i], pr[i], sq);
		for (int i = tid; i < K; i += blockDim.x) sk = fmaf(pr[Q + i], pr[Q + i], sk);
		sq = warp_sum(sq), sk = warp_sum(sk);
		if (lane == 0) red[0][warp] = sq, red[1][warp] = sk;
	}
	__syncthreads();
	float rq = 1.f, rk = 1.f;
	if (a.qw && !a.per_head) {
		sq = sk = 0.f;
		for (int w = 0; w < (int)(blockDim.x >> 5); ++w) sq += red[0][w], sk += red[1][w];
		rq = 1.f / sqrtf(sq / (float)Q + a.eps), rk = 1.f / sqrtf(sk / (float)K + a.eps);
	}
	float* kd = a.kc + row * K;
	for (int e = tid; e < Q + K; e += blockDim.x) {
		const bool isq = e < Q;
		const int c = isq ? e : e - Q, d = c % a.dim;
		const bf16* w = isq ? a.qw : a.kw;
		const float r = a.per_head && w ? rh[e / a.dim] : isq ? rq : rk; // e / dim: query heads, then key heads
		const float* src = pr + (isq ? 0 : Q);
		const int wo = a.per_head ? c - d : 0; // a weight shared by the heads is indexed by the channel inside the head
		float v = src[c] * r * (w ? ldf(w + c - wo) : 1.f);
		if (d < a.rot_dims) {
			const int i = d < half ? d : d - half, o = d < half ? c + half : c - half;
			const float other = src[o] * r * (w ? ldf(w + o - wo) : 1.f);
			v = d < half ? v * cs[i] - other * cs[half + i] : v * cs[i] + other * cs[half + i];
		}
		if (isq) a.q[(size_t)n * Q + c] = v;
		else kd[c] = v;
	}
	float* vd = a.vc + row * Vn;
	if (a.v_norm) { // one warp per value head
		for (int g = warp; g < a.kv_heads; g += (int)(blockDim.x >> 5)) {
			const float* src = pr + Q + K + g * a.vdim;
			float ss = 0.f;
			for (int i = lane; i < a.vdim; i += 32) ss = fmaf(src[i], src[i], ss);
			ss = warp_sum(ss);
			const float rv = 1.f / sqrtf(ss / (float)a.vdim + a.eps);
			for (int i = lane; i < a.vdim; i += 32) vd[g * a.vdim + i] = src[i] * rv;
		}
		return;
	}
	for (int i = tid; i < Vn; i += blockDim.x) vd[i] = pr[Q + K + i];
}

// ---------------------------------------------------------------- routed experts
// Router: per token the `top` highest-scoring experts (lowest index wins a tie) and a softmax restricted to their scores.  One warp per token.
// mode 1: scores are a softmax over ALL `experts` router outputs; the choice is made on score + correction (bf16 [experts] or null), the
// weights are the chosen scores times `scale`, not renormalised.  mode 2: scores are sigmoid(output), choice and weight alike.
__device__ __forceinline__ void moe_route_token(int n, int lane, const float* logits, int ld, int experts, int top, int* sel, float* wt, int mode, const bf16* correction, float scale) {
	const float* z = logits + (size_t)n * ld;
	if (mode == 1) {
		float mx = -INFINITY;
		for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, z[e]);
		mx = warp_max(mx);
		float den = 0.f;
		for (int e = lane; e < experts; e += 32) den += expf(z[e] - mx);
		den = warp_sum(den);
		for (int k = 0; k < top; ++k) {
			float bv = -INFINITY, bs = 0.f;
			int bi = 0x7fffffff;
			for (int e = lane; e < experts; e += 32) {
				bool taken = false;
				for (int j = 0; j < k; ++j) taken |= sel[(size_t)n * top + j] == e;
				const float sc = expf(z[e] - mx) / den, c = sc + (correction ? ldf(correction + e) : 0.f);
				if (!taken && c > bv) bv = c, bi = e, bs = sc;
			}
			for (int o = 16; o > 0; o >>= 1) {
				const float ov = __shfl_xor_sync(0xffffffffu, bv, o), os = __shfl_xor_sync(0xffffffffu, bs, o);
				const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
				if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi, bs = os;
			}
			if (lane == 0) sel[(size_t)n * top + k] = bi, wt[(size_t)n * top + k] = bs * scale;
			__syncwarp();
		}
		return;
	}
	if (mode == 2) { // scores sigmoid(z); the `top` largest, each weighted by its own score
		for (int k = 0; k < top; ++k) {
			float bv = -INFINITY;
			int bi = 0x7fffffff;
			for (int e = lane; e < experts; e += 32) {
				bool taken = false;
				for (int j = 0; j < k; ++j) taken |= sel[(size_t)n * top + j] == e;
				const float sc = sigmoidf_(z[e]);
				if (!taken && sc > bv) bv = sc, bi = e;
			}
			for (int o = 16; o > 0; o >>= 1) {
				const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
				const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
				if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
			}
			if (lane == 0) sel[(size_t)n * top + k] = bi, wt[(size_t)n * top + k] = bv * scale;
			__syncwarp();
		}
		return;
	}
	float first = 0.f, sum = 0.f;
	for (int k = 0; k < top; ++k) {
		float bv = -INFINITY;
		int bi = 0x7fffffff;
		for (int e = lane; e < experts; e += 32) {
			bool taken = false;
			for (int j = 0; j < k; ++j) taken |= sel[(size_t)n * top + j] == e; // written by lane 0 below, visible after the warp barrier
			if (!taken && z[e] > bv) bv = z[e], bi = e;
		}
		for (int o = 16; o > 0; o >>= 1) {
			const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
			const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
			if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
		}
		if (k == 0) first = bv;
		const float p = expf(bv - first); // the first chosen logit is the largest: the softmax's maximum
		sum += p;
		if (lane == 0) sel[(size_t)n * top + k] = bi, wt[(size_t)n * top + k] = p;
		__syncwarp();
	}
	for (int k = lane; k < top; k += 32) wt[(size_t)n * top + k] /= sum;
}
__global__ void k_seq_moe_route(const float* logits, int ld, int experts, int top, int N, int* sel, float* wt, int mode, const bf16* correction, float scale) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int n = blockIdx.x * (blockDim.x >> 5) + warp;
	if (n >= N) return;
	moe_route_token(n, lane, logits, ld, experts, top, sel, wt, mode, correction, scale);
}
// Few tokens (a decode step): routing and grouping in ONE CTA.  The warps route the tokens, then thread e places expert e's pairs in
// token order behind those of the lower experts (same result as k_seq_moe_route followed by k_seq_moe_group).
#define MOE_SMALL_TOKENS 64
__global__ void __launch_bounds__(256) k_seq_moe_route_group(const float* logits, int ld, int experts, int top, int N, int* sel, float* wt, int mode, const bf16* correction, float scale,
                                                             int* seg, int* perm, int* inv) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	for (int n = warp; n < N; n += 8) moe_route_token(n, lane, logits, ld, experts, top, sel, wt, mode, correction, scale);
	__syncthreads();
	const int pairs = N * top;
	for (int e = threadIdx.x; e < experts; e += 256) {
		int below = 0;
		for (int i = 0; i < pairs; ++i) below += sel[i] < e;
		seg[e] = below;
		if (e == experts - 1) seg[experts] = pairs;
		for (int i = 0; i < pairs; ++i)
			if (sel[i] == e) perm[below] = i, inv[i] = below, ++below;
	}
}
// Groups the (token, choice) pairs by expert, pairs of one expert in token order: one CTA per expert counts the pairs of lower
// experts (its group's first row) and places its own.  seg[e] .. seg[e+1] are expert e's rows, perm[row] = pair, inv[pair] = row.
__global__ void __launch_bounds__(256) k_seq_moe_group(const int* sel, int pairs, int experts, int* seg, int* perm, int* inv) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	__shared__ int wsum[8], base_s, run_s;
	const int e = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
	int below = 0;
	for (int i = tid; i < pairs; i += 256) below += sel[i] < e;
	for (int o = 16; o > 0; o >>= 1) below += __shfl_xor_sync(0xffffffffu, below, o);
	if (lane == 0) wsum[warp] = below;
	__syncthreads();
	if (tid == 0) {
		int s = 0;
		for (int w = 0; w < 8; ++w) s += wsum[w];
		base_s = s, run_s = 0;
		seg[e] = s;
		if (e == experts - 1) seg[experts] = pairs;
	}
	__syncthreads();
	const int base = base_s;
	for (int i0 = 0; i0 < pairs; i0 += 256) {
		const int i = i0 + tid;
		const bool mine = i < pairs && sel[i] == e;
		const unsigned bal = __ballot_sync(0xffffffffu, mine);
		__syncthreads(); // the previous pass's readers of wsum / run_s are done
		if (lane == 0) wsum[warp] = __popc(bal);
		__syncthreads();
		int before = run_s;
		for (int w = 0; w < warp; ++w) before += wsum[w];
		if (mine) {
			const int r = base + before + __popc(bal & ((1u << lane) - 1));
			perm[r] = i, inv[i] = r;
		}
		__syncthreads();
		if (tid == 0) {
			int s = run_s;
			for (int w = 0; w < 8; ++w) s += wsum[w];
			run_s = s;
		}
	}
}
// rows of the grouped activation matrix: Xp[row] = h[perm[row] / top]
template <typename AT>
__global__ void k_seq_moe_gather(AT* xp, const AT* h, const int* perm, int top, int pairs, int width) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= (size_t)pairs * width) return;
	const size_t r = i / width, c = i % width;
	xp[i] = h[(size_t)(perm[r] / top) * width + c];
}
// x[n] += (res ? res[n] : 0) + sum_k wt[n][k] * y[inv[n * top + k]]   (choices in order of rank; `store`: x[n] = the sum alone)
// A choice sel >= real is an identity expert: its output is the token's own input row h[n].
template <typename AT>
__global__ void k_seq_moe_combine(float* x, const float* res, const float* y, const int* inv, const float* wt, int top, int N, int width, const int* sel, int real, const AT* h,
                                  int store) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= (size_t)N * width) return;
	const size_t n = i / width, c = i % width;
	float s = 0.f;
	for (int k = 0; k < top; ++k) {
		const float v = sel[n * top + k] >= real ? ldf(h + i) : y[(size_t)inv[n * top + k] * width + c];
		s = fmaf(wt[n * top + k], v, s);
	}
	if (store) x[i] = s;
	else x[i] += res ? res[i] + s : s;
}

// ---------------------------------------------------------------- hyper-connections: several copies of the residual stream
// x is [N][streams][width].  Read: u = sum_s in[s] x_s (in == null: every stream counts once), then the RMS norm of u with a weight
// per column (w_len = width) or one number for all (w_len = 1); one CTA per row, rows[] picks tokens (the rows whose logits are wanted).
template <typename AT>
__global__ void __launch_bounds__(256) k_seq_hc_read(AT* out, const float* x, const int* rows, const bf16* in, const bf16* w, int w_len, float offset, float eps, int R, int width,
                                                     int streams) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	__shared__ float red[8];
	const int tid = threadIdx.x, nt = blockDim.x, r = blockIdx.x;
	const float* src = x + (size_t)(rows ? rows[r] : r) * streams * width;
	auto mixed = [&](int c) {
		float u = 0.f;
		for (int s = 0; s < streams; ++s) u = fmaf(in ? ldf(in + s) : 1.f, src[(size_t)s * width + c], u);
		return u;
	};
	float keep[RMS_KEEP];
	float ss = 0.f;
#pragma unroll
	for (int i = 0; i < RMS_KEEP; ++i) {
		const int c = i * nt + tid;
		keep[i] = c < width ? mixed(c) : 0.f;
		ss = fmaf(keep[i], keep[i], ss);
	}
	for (int c = RMS_KEEP * nt + tid; c < width; c += nt) {
		const float u = mixed(c);
		ss = fmaf(u, u, ss);
	}
	ss = warp_sum(ss);
	if ((tid & 31) == 0) red[tid >> 5] = ss;
	__syncthreads();
	ss = 0.f;
	for (int i = 0; i < (nt >> 5); ++i) ss += red[i];
	const float rinv = 1.f / sqrtf(ss / (float)width + eps);
	AT* d = out + (size_t)r * width;
#pragma unroll
	for (int i = 0; i < RMS_KEEP; ++i) {
		const int c = i * nt + tid;
		if (c < width) d[c] = to_act<AT>(keep[i] * rinv * (ldf(w + (w_len == 1 ? 0 : c)) + offset));
	}
	for (int c = RMS_KEEP * nt + tid; c < width; c += nt) d[c] = to_act<AT>(mixed(c) * rinv * (ldf(w + (w_len == 1 ? 0 : c)) + offset));
}
// Write: x_t <- sum_s mix[s][t] x_s + out[t] y for every stream t at once, from the old streams.  y = base (the sublayer's last product,
// or null) + the routed experts' weighted sum when `moe.y` is set (choices in order of rank; identity experts return the input row h).
#define HC_MAX 16
struct HcMoe {
	const float* y;  // [pairs][width] grouped expert outputs, or null: no routed part
	const int* inv;
	const int* sel;
	const float* wt;
	int top, real;
};
// One CTA per token.  When `rd.out` is set the same pass also forms the NEXT sublayer's input from the streams it has just written
// (u = sum_t in[t] x_t, RMS norm, weight), so the streams are not read again: hc_write followed by hc_read in one kernel.  The row of h
// that identity experts read may be the very row rd.out overwrites: all reads of it come before the barrier, all writes after.
struct HcRead {
	void* out;       // [N][width] of the activation type, or null: write only
	const bf16* in;  // [streams]
	const bf16* w;
	int w_len;
	float offset, eps;
};
// (a thread's columns alternate loads and stores of the same matrix, which do not overlap in time, so a thread should have one
// group of columns, or few)
#define HC_KEEP 4
template <int V>
struct HcVec { float v[V]; };
template <int V>
__device__ __forceinline__ HcVec<V> hc_load(const float* p) {
	HcVec<V> r;
	if constexpr (V == 4) {
		const float4 t = *(const float4*)p;
		r.v[0] = t.x, r.v[1] = t.y, r.v[2] = t.z, r.v[3] = t.w;
	} else r.v[0] = *p;
	return r;
}
template <int V>
__device__ __forceinline__ void hc_store(float* p, const HcVec<V>& r) {
	if constexpr (V == 4) *(float4*)p = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
	else *p = r.v[0];
}
// V = 4: width is a multiple of 4 and a thread owns four neighbouring columns (16-byte loads and stores); V = 1: any width.
// SM: the most streams this instance holds in registers (4 or HC_MAX)
template <typename AT, int V, int SM>
__global__ void __launch_bounds__(V == 4 ? 512 : 1024) k_seq_hc_write(float* x, const float* base, const bf16* mix, const bf16* outw, int N, int width, int streams, HcMoe moe, const AT* h, HcRead rd) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	__shared__ float red[32];
	const int tid = threadIdx.x, nt = blockDim.x;
	const size_t n = blockIdx.x;
	// the few coefficients (mix, out, the next read's in) are read where they are used: every lane the same address, served by L1; no
	// staging and no barrier before the first loads of the streams go out
	auto c_mix = [&](int s, int t) { return ldf(mix + s * streams + t); };
	auto c_out = [&](int t) { return ldf(outw + t); };
	auto c_in = [&](int t) { return rd.out ? ldf(rd.in + t) : 0.f; };
	float* xr = x + n * streams * width;
	auto column = [&](int c) { // writes the new streams of columns c .. c + V - 1, returns the next read's weighted sum of them
		const size_t i = n * width + c;
		HcVec<V> y;
#pragma unroll
		for (int e = 0; e < V; ++e) y.v[e] = 0.f;
		if (base) y = hc_load<V>(base + i);
		if (moe.y) {
			HcVec<V> sacc;
#pragma unroll
			for (int e = 0; e < V; ++e) sacc.v[e] = 0.f;
			for (int k = 0; k < moe.top; ++k) {
				HcVec<V> v;
				if (moe.sel[n * moe.top + k] >= moe.real) {
#pragma unroll
					for (int e = 0; e < V; ++e) v.v[e] = ldf(h + i + e);
				} else v = hc_load<V>(moe.y + (size_t)moe.inv[n * moe.top + k] * width + c);
				const float wk = moe.wt[n * moe.top + k];
#pragma unroll
				for (int e = 0; e < V; ++e) sacc.v[e] = fmaf(wk, v.v[e], sacc.v[e]);
			}
#pragma unroll
			for (int e = 0; e < V; ++e) y.v[e] += sacc.v[e];
		}
		HcVec<V> old[SM];
#pragma unroll
		for (int s = 0; s < SM; ++s)
			if (s < streams) old[s] = hc_load<V>(xr + (size_t)s * width + c);
		HcVec<V> u;
#pragma unroll
		for (int e = 0; e < V; ++e) u.v[e] = 0.f;
		for (int t = 0; t < streams; ++t) {
			HcVec<V> v;
#pragma unroll
			for (int e = 0; e < V; ++e) v.v[e] = 0.f;
#pragma unroll
			for (int s = 0; s < SM; ++s)
				if (s < streams) {
					const float mx = c_mix(s, t);
#pragma unroll
					for (int e = 0; e < V; ++e) v.v[e] = fmaf(mx, old[s].v[e], v.v[e]);
				}
			const float co = c_out(t), ci = c_in(t);
#pragma unroll
			for (int e = 0; e < V; ++e) v.v[e] = fmaf(co, y.v[e], v.v[e]), u.v[e] = fmaf(ci, v.v[e], u.v[e]);
			hc_store<V>(xr + (size_t)t * width + c, v);
		}
		return u;
	};
	HcVec<V> keep[HC_KEEP];
	float ss = 0.f;
#pragma unroll
	for (int i = 0; i < HC_KEEP; ++i) {
		const int c = (i * nt + tid) * V;
		if (c < width) keep[i] = column(c);
		else {
#pragma unroll
			for (int e = 0; e < V; ++e) keep[i].v[e] = 0.f;
		}
#pragma unroll
		for (int e = 0; e < V; ++e) ss = fmaf(keep[i].v[e], keep[i].v[e], ss);
	}
	for (int c = (HC_KEEP * nt + tid) * V; c < width; c += nt * V) {
		const HcVec<V> u = column(c);
#pragma unroll
		for (int e = 0; e < V; ++e) ss = fmaf(u.v[e], u.v[e], ss);
	}
	if (!rd.out) return;
	ss = warp_sum(ss);
	if ((tid & 31) == 0) red[tid >> 5] = ss;
	__syncthreads();
	ss = 0.f;
	for (int i = 0; i < (nt >> 5); ++i) ss += red[i];
	const float rinv = 1.f / sqrtf(ss / (float)width + rd.eps);
	AT* d = (AT*)rd.out + n * width;
#pragma unroll
	for (int i = 0; i < HC_KEEP; ++i) {
		const int c = (i * nt + tid) * V;
		if (c < width) {
#pragma unroll
			for (int e = 0; e < V; ++e) d[c + e] = to_act<AT>(keep[i].v[e] * rinv * (ldf(rd.w + (rd.w_len == 1 ? 0 : c + e)) + rd.offset));
		}
	}
	for (int c = (HC_KEEP * nt + tid) * V; c < width; c += nt * V) { // wider rows: the sum is formed again from the streams just written (by this thread)
#pragma unroll
		for (int e = 0; e < V; ++e) {
			float u = 0.f;
			for (int t = 0; t < streams; ++t) u = fmaf(c_in(t), xr[(size_t)t * width + c + e], u);
			d[c + e] = to_act<AT>(u * rinv * (ldf(rd.w + (rd.w_len == 1 ? 0 : c + e)) + rd.offset));
		}
	}
}
// Post-norm blocks: x[n] += y / sqrt(mean(y^2) + eps) * (w + offset), where y = base (a sublayer's last product, or null) + the routed
// experts' sum when `moe.y` is set (choices in order of rank, each times its weight, or times one when moe.wt is null: the weight went
// in at the expert's input).  The same pass writes the new row of x in the activation type: the input of the sublayer that follows.
// One CTA per token.  V = 4: width is a multiple of 4 and a thread owns groups of four neighbouring columns (16-byte loads and stores);
// V = 1: any width.  A thread keeps PN_KEEP groups of y in registers (wider rows form y a second time).
#define PN_KEEP 4
template <typename AT, int V>
__device__ __forceinline__ void pn_store_act(AT* p, const HcVec<V>& r) {
	if constexpr (V == 4 && sizeof(AT) == 2) {
		__nv_bfloat162 lo = __floats2bfloat162_rn(r.v[0], r.v[1]), hi = __floats2bfloat162_rn(r.v[2], r.v[3]);
		uint2 u;
		u.x = *reinterpret_cast<unsigned*>(&lo), u.y = *reinterpret_cast<unsigned*>(&hi);
		*reinterpret_cast<uint2*>(p) = u;
	} else {
#pragma unroll
		for (int e = 0; e < V; ++e) p[e] = to_act<AT>(r.v[e]);
	}
}
template <typename AT, int V>
__global__ void __launch_bounds__(256) k_seq_post_norm(float* x, AT* act, const float* base, HcMoe moe, const bf16* w, float offset, float eps, int N, int width) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	__shared__ float red[8];
	const int tid = threadIdx.x, nt = blockDim.x;
	const size_t n = blockIdx.x;
	auto yval = [&](int c) {
		HcVec<V> y;
#pragma unroll
		for (int e = 0; e < V; ++e) y.v[e] = 0.f;
		if (base) y = hc_load<V>(base + n * width + c);
		if (moe.y)
			for (int k = 0; k < moe.top; ++k) {
				const HcVec<V> v = hc_load<V>(moe.y + (size_t)moe.inv[n * moe.top + k] * width + c);
				const float wk = moe.wt ? moe.wt[n * moe.top + k] : 1.f;
#pragma unroll
				for (int e = 0; e < V; ++e) y.v[e] = moe.wt ? fmaf(wk, v.v[e], y.v[e]) : y.v[e] + v.v[e];
			}
		return y;
	};
	HcVec<V> keep[PN_KEEP];
	float ss = 0.f;
#pragma unroll
	for (int i = 0; i < PN_KEEP; ++i) {
		const int c = (i * nt + tid) * V;
		if (c < width) keep[i] = yval(c);
		else {
#pragma unroll
			for (int e = 0; e < V; ++e) keep[i].v[e] = 0.f;
		}
#pragma unroll
		for (int e = 0; e < V; ++e) ss = fmaf(keep[i].v[e], keep[i].v[e], ss);
	}
	for (int c = (PN_KEEP * nt + tid) * V; c < width; c += nt * V) {
		const HcVec<V> y = yval(c);
#pragma unroll
		for (int e = 0; e < V; ++e) ss = fmaf(y.v[e], y.v[e], ss);
	}
	ss = warp_sum(ss);
	if ((tid & 31) == 0) red[tid >> 5] = ss;
	__syncthreads();
	ss = 0.f;
	for (int i = 0; i < (nt >> 5); ++i) ss += red[i]; // every thread adds the warps' sums in the same order
	const float rinv = 1.f / sqrtf(ss / (float)width + eps);
	float* xr = x + n * width;
	AT* ar = act + n * width;
	auto put = [&](int c, const HcVec<V>& y) {
		HcVec<V> v = hc_load<V>(xr + c);
#pragma unroll
		for (int e = 0; e < V; ++e) v.v[e] += y.v[e] * rinv * (ldf(w + c + e) + offset);
		hc_store<V>(xr + c, v);
		pn_store_act<AT, V>(ar + c, v);
	};
#pragma unroll
	for (int i = 0; i < PN_KEEP; ++i) {
		const int c = (i * nt + tid) * V;
		if (c < width) put(c, keep[i]);
	}
	for (int c = (PN_KEEP * nt + tid) * V; c < width; c += nt * V) put(c, yval(c));
}
// out[n] = sum of the streams of token n
__global__ void k_seq_stream_sum(float* out, const float* x, int N, int width, int streams) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= (size_t)N * width) return;
	const size_t n = i / width, c = i % width;
	float v = 0.f;
	for (int s = 0; s < streams; ++s) v += x[(n * streams + s) * width + c];
	out[i] = v;
}

// ---------------------------------------------------------------- linear recurrences served by the gated-linear-attention scan
// mLSTM, HGRN2 and Mamba-2 are all S <- diag(a) S + k v^T, o = S^T q per head; what differs is how a, k, v, q come out of the
// projection and what happens to o.  A preparation kernel writes them as the scan's input (`lin`: rows [q | k | v] per token, and
// the decay matrix), the scan itself is k_seq_gla_scan, k_seq_lin_out finishes.

// mLSTM gates.  Per (sequence, head), over the step's tokens in order, with the running maximum m carried in the slot state:
//   li = cap tanh((i_raw) / cap), lf = logsigmoid(cap tanh(f_raw / cap)), m_t = max(lf + m_(t-1), li),
//   keep_t = exp(lf + m_(t-1) - m_t), take_t = exp(li - m_t).
// One warp per (sequence, head), 32 tokens per round: with F the running sum of lf inside the round, m_t = F_t + max(m_in, max_(s<=t)(li_s - F_s)).
struct MlstmGates {
	const float* proj; // biased projection; raw gates at columns icol + h, fcol + h
	int ldp, icol, fcol, heads;
	float cap;
	float* m_state;    // [slots][heads]
	float* keep;       // [N][heads]
	float* take;       // [N][heads]
	float* m_out;      // [N][heads]
};
__global__ void k_seq_mlstm_gates(MlstmGates a, SeqBatch sb) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const int b = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
	const int start = sb.sstart[b], cnt = sb.scount[b];
	float* mp = a.m_state + (size_t)sb.sslot[b] * a.heads + h;
	float m_in = *mp;
	for (int t0 = 0; t0 < cnt; t0 += 32) {
		const int t = t0 + lane;
		const bool live = t < cnt;
		float li = -INFINITY, lf = 0.f;
		if (live) {
			const float* pr = a.proj + (size_t)(start + t) * a.ldp;
			li = a.cap * tanhf(pr[a.icol + h] / a.cap);
			const float fr = a.cap * tanhf(pr[a.fcol + h] / a.cap);
			lf = -softplusf_(-fr);
		}
		// the two scans run in double: a round's sum of log forget gates can reach hundreds, where a float keeps four decimals only
		double F = lf;
		for (int o = 1; o < 32; o <<= 1) {
			const double up = __shfl_up_sync(0xffffffffu, F, o);
			if (lane >= o) F += up;
		}
		double A = live ? (double)li - F : -INFINITY;
		for (int o = 1; o < 32; o <<= 1) {
			const double up = __shfl_up_sync(0xffffffffu, A, o);
			if (lane >= o) A = fmax(A, up);
		}
		const double m = F + fmax((double)m_in, A);
		double m_prev = __shfl_up_sync(0xffffffffu, m, 1);
		if (lane == 0) m_prev = m_in;
		if (live) {
			const size_t o = (size_t)(start + t) * a.heads + h;
			a.keep[o] = expf((float)((double)lf + m_prev - m)), a.take[o] = expf((float)((double)li - m)), a.m_out[o] = (float)m;
		}
		m_in = (float)__shfl_sync(0xffffffffu, m, min(31, cnt - t0 - 1));
	}
	if (lane == 0) *mp = m_in;
}

// Scan input of one token and head.  lin row: [q: heads*dim | k: heads*dim | v: heads*vs], decay row: [heads*dim].
//   LIN_MLSTM : q, k as projected; v' = take * [v, 1, 0..] (vs = vdim rounded up past one extra column: the normaliser n rides as a value
//               column of ones); decay = keep for every channel.
//   LIN_HGRN2 : q = silu(q_raw); f = l + (1 - l) sigmoid(f_raw); k = 1 - f; decay = f; v as projected.
//   LIN_MAMBA2: q = C and k = B of the head's group (after the convolution); dt = softplus(dt_raw + dt_bias); v' = dt x; decay = exp(-exp(A_log) dt).
enum { LIN_MLSTM = 0, LIN_HGRN2 = 1, LIN_MAMBA2 = 2 };
struct LinPack {
	int mode;
	const float* proj;
	int ldp, qcol, kcol, vcol; // HGRN2: kcol = the raw forget gate's column
	const float *keep, *take;  // LIN_MLSTM
	const bf16* lower;         // LIN_HGRN2
	const float *xs, *bs, *cs; // LIN_MAMBA2: convolved x [N][heads*vdim], B and C [N][groups*dim]
	int dtcol, groups;
	const bf16 *dt_bias, *a_log;
	float* lin;
	float* decay;
	int heads, dim, vdim, vs;
};
__global__ void k_seq_lin_pack(LinPack a, int N) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const int n = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, H = a.heads, D = a.dim, V = a.vdim;
	const int ldl = 2 * H * D + H * a.vs;
	const float* pr = a.proj + (size_t)n * a.ldp;
	float* lq = a.lin + (size_t)n * ldl + h * D;
	float* lk = lq + H * D;
	float* lv = a.lin + (size_t)n * ldl + 2 * H * D + h * a.vs;
	float* dc = a.decay + ((size_t)n * H + h) * D;
	if (a.mode == LIN_MLSTM) {
		const float keep = a.keep[(size_t)n * H + h], take = a.take[(size_t)n * H + h];
		for (int i = tid; i < D; i += blockDim.x) lq[i] = pr[a.qcol + h * D + i], lk[i] = pr[a.kcol + h * D + i], dc[i] = keep;
		for (int i = tid; i < a.vs; i += blockDim.x) lv[i] = i < V ? take * pr[a.vcol + h * V + i] : i == V ? take : 0.f;
	} else if (a.mode == LIN_HGRN2) {
		for (int i = tid; i < D; i += blockDim.x) {
			const float q = pr[a.qcol + h * D + i], l = ldf(a.lower + h * D + i);
			const float f = l + (1.f - l) * sigmoidf_(pr[a.kcol + h * D + i]);
			lq[i] = q * sigmoidf_(q), lk[i] = 1.f - f, dc[i] = f;
		}
		for (int i = tid; i < a.vs; i += blockDim.x) lv[i] = i < V ? pr[a.vcol + h * V + i] : 0.f;
	} else {
		const int g = h / (H / a.groups);
		const float dt = softplusf_(pr[a.dtcol + h] + ldf(a.dt_bias + h));
		const float dec = expf(-expf(ldf(a.a_log + h)) * dt);
		for (int i = tid; i < D; i += blockDim.x) {
			lq[i] = a.cs[((size_t)n * a.groups + g) * D + i], lk[i] = a.bs[((size_t)n * a.groups + g) * D + i], dc[i] = dec;
		}
		for (int i = tid; i < a.vs; i += blockDim.x) lv[i] = i < V ? dt * a.xs[((size_t)n * H + h) * V + i] : 0.f;
	}
}

// Read-out of a linear recurrence.  The token's heads*vdim outputs (o[n*ldo + h*ohs + d]) are taken in units of `unit` columns (vdim: per
// head; heads*vdim / groups: equal parts); one warp per (token, unit):
//   mLSTM (m_t given): o /= max(|o[.., vdim]|, exp(-m_t)) + 1e-6 first (column vdim of the head holds n . q);
//   skip given: o += skip_w[h] * skip[n][h*vdim + d];   gate_mode 3: o *= silu(gate) BEFORE the norm;
//   then RMS over the unit (eps inside the root), times w[col % w_mod] (null: no weight), times sigmoid(gate) (gate_mode 1), times mul.
struct LinOut {
	const float* o;
	int ldo, ohs, heads, vdim, unit;
	const bf16* w;
	int w_mod;
	const float* gate;
	int ldg, gate_mode;
	const float* m_t;     // [N][heads] or null
	const float* skip;    // [N][heads*vdim] or null
	const bf16* skip_w;   // [heads]
	float eps, mul;
};
template <typename AT>
__global__ void k_seq_lin_out(AT* out, LinOut a, int N) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int inner = a.heads * a.vdim, units = inner / a.unit;
	const size_t u = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
	if (u >= (size_t)N * units) return;
	const size_t n = u / units;
	const int c0 = (int)(u % units) * a.unit;
	// a unit that is one head (mLSTM, HGRN2): the head, its row of o and the mLSTM's denominator are the same for the whole warp
	const bool one_head = a.unit == a.vdim;
	const int h0 = c0 / a.vdim;
	auto denominator = [&](int h) { return fmaxf(fabsf(a.o[n * a.ldo + (size_t)h * a.ohs + a.vdim]), expf(-a.m_t[n * a.heads + h])) + 1e-6f; };
	const float den0 = a.m_t && one_head ? denominator(h0) : 1.f;
	auto value = [&](int c) {
		const int h = one_head ? h0 : c / a.vdim, d = one_head ? c - c0 : c % a.vdim;
		const float* oh = a.o + n * a.ldo + (size_t)h * a.ohs;
		float v = oh[d];
		if (a.m_t) v /= one_head ? den0 : denominator(h);
		if (a.skip) v = fmaf(ldf(a.skip_w + h), a.skip[n * inner + c], v);
		if (a.gate_mode == 3) {
			const float g = a.gate[n * a.ldg + c];
			v *= g * sigmoidf_(g);
		}
		return v;
	};
	// two passes over the unit, both straight from memory: holding the values in registers between them was measured slower (the
	// unrolled rounds cost more than the second read, which comes from L1 / L2)
	float ss = 0.f;
	for (int i = lane; i < a.unit; i += 32) {
		const float v = value(c0 + i);
		ss = fmaf(v, v, ss);
	}
	ss = warp_sum(ss);
	const float r = 1.f / sqrtf(ss / (float)a.unit + a.eps) * a.mul;
	for (int i = lane; i < a.unit; i += 32) {
		const int c = c0 + i;
		float v = value(c) * r;
		if (a.w) v *= ldf(a.w + c % a.w_mod);
		if (a.gate_mode == 1) v *= sigmoidf_(a.gate[n * a.ldg + c]);
		out[n * inner + c] = to_act<AT>(v);
	}
}

// ---------------------------------------------------------------- products  Y[n][m] = sum_k X[n][k] W[m][k]
// blockIdx.z = batch (per-head products): X, W, Y advance by xbs, wbs, ybs elements.
enum { EPI_F32 = 0, EPI_ACT = 1, EPI_DYT_RES = 2, EPI_RES = 3, EPI_ACT_RELU2 = 4, EPI_DECAY = 5 };
struct GemmArgs {
	const void* X;
	long ldx, xbs;
	const bf16* W;
	long ldw, wbs;
	void* Y;
	long ldy, ybs;
	int N, M, K;
	int epi;                 // EPI_F32: Y fp32; EPI_ACT: Y of the activation type; EPI_DYT_RES: Y fp32 residual += tanh(alpha acc) w + b;
	                         // EPI_RES: Y fp32 residual += (res ? res : 0) + acc; EPI_ACT_RELU2: Y of the activation type = relu(acc)^2;
	                         // EPI_DECAY: Y fp32 = sigmoid(acc)^epi_f = exp(-softplus(-acc) * epi_f)
	float epi_f;
	const bf16 *nw, *nb, *na;
	int w_immutable;         // W is a model weight: it may be read before the previous kernel has finished (products of gathered keys set 0)
	const bf16* bias;        // [batch][M] or null: added to the accumulator first
	const float* res;        // EPI_RES: a second addend laid out like Y, or null
	const float* gate;       // EPI_ACT: the output is multiplied by sigmoid(gate[z * gbs + n * ldgate + m]); null: none
	long ldgate, gbs;
	const int* seg;          // grouped products: batch z owns rows [seg[z], seg[z+1]) of X and Y (xbs = ybs = 0), N bounds one group; null: none
	int x_rows;              // grouped products: rows of X and Y over all groups
	int split;               // > 0: output columns m >= split leave in the activation type to Y2[n][m - split] (row stride ldy2), whatever epi says:
	int split_act = 0;       //      as relu(acc)^2 (0) or as they are (1)
	void* Y2;
	long ldy2;
	float out_scale = 0.f;   // != 0: the accumulator (after the bias) is multiplied by it
	const float* rs = nullptr; // a factor per row on the accumulator (after the bias): rs[(rs_idx ? rs_idx[row] : row) * rs_ld], through a sigmoid when rs_act is 1
	const int* rs_idx = nullptr;
	long rs_ld = 1;
	int rs_act = 0;
};
// rows of batch z: first row and count
struct GemmRows {
	int base, count;
};
__device__ __forceinline__ GemmRows gemm_rows(const GemmArgs& a, int z) {
	if (!a.seg) return GemmRows{0, a.N};
	const int b = a.seg[z];
	return GemmRows{b, a.seg[z + 1] - b};
}
template <typename AT>
__device__ __forceinline__ void gemm_store(const GemmArgs& a, int z, const GemmRows& gr, int n, int m, float acc) {
	if (n >= gr.count || m >= a.M) return;
	const size_t o = (size_t)z * a.ybs + (size_t)(gr.base + n) * a.ldy + m;
	if (a.bias) acc += ldf(a.bias + (size_t)z * a.M + m);
	if (a.out_scale != 0.f) acc *= a.out_scale;
	if (a.rs) {
		const float f = a.rs[(size_t)(a.rs_idx ? a.rs_idx[gr.base + n] : gr.base + n) * a.rs_ld];
		acc *= a.rs_act ? sigmoidf_(f) : f;
	}
	if (a.split > 0 && m >= a.split) {
		const float r = fmaxf(acc, 0.f);
		((AT*)a.Y2)[(size_t)(gr.base + n) * a.ldy2 + (m - a.split)] = to_act<AT>(a.split_act ? acc : r * r);
		return;
	}
	if (a.epi == EPI_F32) ((float*)a.Y)[o] = acc;
	else if (a.epi == EPI_ACT) {
		if (a.gate) acc *= sigmoidf_(a.gate[(size_t)z * a.gbs + (size_t)(gr.base + n) * a.ldgate + m]);
		((AT*)a.Y)[o] = to_act<AT>(acc);
	} else if (a.epi == EPI_RES) ((float*)a.Y)[o] += a.res ? a.res[o] + acc : acc;
	else if (a.epi == EPI_DECAY) ((float*)a.Y)[o] = expf(-softplusf_(-acc) * a.epi_f);
	else if (a.epi == EPI_ACT_RELU2) {
		const float r = fmaxf(acc, 0.f);
		((AT*)a.Y)[o] = to_act<AT>(r * r);
	} else ((float*)a.Y)[o] += tanhf(ldf(a.na) * acc) * ldf(a.nw + m) + ldf(a.nb + m);
}

// exact mode: fp32 FMA, 64 x 64 tile, 16-deep steps, 256 threads with 4 x 4 outputs each
__global__ void __launch_bounds__(256) k_seq_gemm_f32(GemmArgs a) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	__shared__ float Xs[16][64 + 4], Ws[16][64 + 4];
	const int z = blockIdx.z, n0 = blockIdx.y * 64, m0 = blockIdx.x * 64, tid = threadIdx.x;
	const GemmRows gr = gemm_rows(a, z);
	if (n0 >= gr.count) return;
	const float* X = (const float*)a.X + (size_t)z * a.xbs + (size_t)gr.base * a.ldx;
	const bf16* W = a.W + (size_t)z * a.wbs;
	const int tn = (tid / 16) * 4, tm = (tid % 16) * 4;
	float acc[4][4] = {};
	for (int k0 = 0; k0 < a.K; k0 += 16) {
		for (int i = tid; i < 64 * 16; i += 256) {
			const int r = i / 16, k = i % 16;
			Xs[k][r] = (n0 + r < gr.count && k0 + k < a.K) ? X[(size_t)(n0 + r) * a.ldx + k0 + k] : 0.f;
			Ws[k][r] = (m0 + r < a.M && k0 + k < a.K) ? ldf(W + (size_t)(m0 + r) * a.ldw + k0 + k) : 0.f;
		}
		__syncthreads();
#pragma unroll
		for (int k = 0; k < 16; ++k) {
			float xv[4], wv[4];
#pragma unroll
			for (int i = 0; i < 4; ++i) xv[i] = Xs[k][tn + i], wv[i] = Ws[k][tm + i];
#pragma unroll
			for (int i = 0; i < 4; ++i)
#pragma unroll
				for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
		}
		__syncthreads();
	}
#pragma unroll
	for (int i = 0; i < 4; ++i)
#pragma unroll
		for (int j = 0; j < 4; ++j) gemm_store<float>(a, z, gr, n0 + tn + i, m0 + tm + j, acc[i][j]);
}

// bf16 x bf16 -> fp32 on the tensor cores for ANY shape (edges are zero-filled in shared memory): 64 tokens x 64 rows per
// CTA, 32-deep steps, four warps of 32 x 32.  The tcgen05 kernel below takes the shapes that fill its tiles.
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&A)[4], const uint32_t (&B)[2]) {
	asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
	             : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
	             : "r"(A[0]), "r"(A[1]), "r"(A[2]), "r"(A[3]), "r"(B[0]), "r"(B[1]));
}
#define GB_LD 40 // bf16 per shared-memory row: 32 + 8 keeps the fragment reads conflict-free
__device__ __forceinline__ void gemm_fill_tile(bf16 (*dst)[GB_LD], const bf16* src, long ld, int r0, int rows, int k0, int K, int tid) {
	// 64 rows x 32 columns as 256 groups of 8: two per thread
	for (int i = tid; i < 256; i += 128) {
		const int r = i >> 2, c = (i & 3) * 8;
		const bf16* p = src + (size_t)(r0 + r) * ld + k0 + c;
		uint4 v = make_uint4(0, 0, 0, 0);
		if (r0 + r < rows) {
			if (k0 + c + 8 <= K && (((uintptr_t)p) & 15) == 0) v = *(const uint4*)p;
			else {
				bf16 t[8];
#pragma unroll
				for (int e = 0; e < 8; ++e) t[e] = k0 + c + e < K ? p[e] : __float2bfloat16_rn(0.f);
				v = *(const uint4*)t;
			}
		}
		*(uint4*)&dst[r][c] = v;
	}
}
__global__ void __launch_bounds__(128) k_seq_gemm_bf16(GemmArgs a) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	__shared__ __align__(16) bf16 Xs[64][GB_LD], Ws[64][GB_LD];
	const int z = blockIdx.z, n0 = blockIdx.y * 64, m0 = blockIdx.x * 64, tid = threadIdx.x;
	const GemmRows gr = gemm_rows(a, z);
	if (n0 >= gr.count) return;
	const bf16* X = (const bf16*)a.X + (size_t)z * a.xbs + (size_t)gr.base * a.ldx;
	const bf16* W = a.W + (size_t)z * a.wbs;
	const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
	const int wn = (warp >> 1) * 32, wm = (warp & 1) * 32;
	float acc[2][4][4] = {};
	for (int k0 = 0; k0 < a.K; k0 += 32) {
		gemm_fill_tile(Xs, X, a.ldx, n0, gr.count, k0, a.K, tid);
		gemm_fill_tile(Ws, W, a.ldw, m0, a.M, k0, a.K, tid);
		__syncthreads();
#pragma unroll
		for (int kk = 0; kk < 32; kk += 16) {
			uint32_t A[2][4], B[4][2];
#pragma unroll
			for (int i = 0; i < 2; ++i) {
				const int r = wn + i * 16 + g;
				A[i][0] = *(const uint32_t*)&Xs[r][kk + 2 * t], A[i][1] = *(const uint32_t*)&Xs[r + 8][kk + 2 * t];
				A[i][2] = *(const uint32_t*)&Xs[r][kk + 2 * t + 8], A[i][3] = *(const uint32_t*)&Xs[r + 8][kk + 2 * t + 8];
			}
#pragma unroll
			for (int j = 0; j < 4; ++j) {
				const int r = wm + j * 8 + g;
				B[j][0] = *(const uint32_t*)&Ws[r][kk + 2 * t], B[j][1] = *(const uint32_t*)&Ws[r][kk + 2 * t + 8];
			}
#pragma unroll
			for (int i = 0; i < 2; ++i)
#pragma unroll
				for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], A[i], B[j]);
		}
		__syncthreads();
	}
#pragma unroll
	for (int i = 0; i < 2; ++i)
#pragma unroll
		for (int j = 0; j < 4; ++j) {
			const int n = n0 + wn + i * 16 + g, m = m0 + wm + j * 8 + 2 * t;
			gemm_store<bf16>(a, z, gr, n, m, acc[i][j][0]), gemm_store<bf16>(a, z, gr, n, m + 1, acc[i][j][1]);
			gemm_store<bf16>(a, z, gr, n + 8, m, acc[i][j][2]), gemm_store<bf16>(a, z, gr, n + 8, m + 1, acc[i][j][3]);
		}
}

// Few tokens (decode): every weight is used once, so the kernel is a stream over W.  A CTA owns 16 weight rows, its warps (8, or 16 when the matrix has few rows)
// take interleaved 32-wide slices of K; a lane loads 16 bytes of row g and of row g + 8 per slice straight into the A
// fragments of two m16n8k16 MMAs (the k order inside a slice is permuted the same way for A and B, which a sum over k does
// not see); tokens are the MMA's N.  The warps' partial tiles are added in warp order through shared memory.
template <int NT, int NW>
__global__ void __launch_bounds__(NW * 32) k_seq_gemm_skinny(GemmArgs a) {
	__shared__ float red[NW][16][NT * 8 + 1];
	const int z = blockIdx.z, m0 = blockIdx.x * 16, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
	bool waited = false;
	pdl_launch_next();
	GemmRows gr{0, a.N};
	if (a.seg) { // the groups come from the previous kernel: a group without rows leaves before it touches its weights
		pdl_wait_prev(), waited = true;
		gr = gemm_rows(a, z);
		if (gr.count == 0) return;
	}
	const bf16* X = (const bf16*)a.X + (size_t)z * a.xbs + (size_t)gr.base * a.ldx;
	const bf16* W = a.W + (size_t)z * a.wbs;
	const bf16* w0 = W + (size_t)min(m0 + g, a.M - 1) * a.ldw;
	const bf16* w1 = W + (size_t)min(m0 + g + 8, a.M - 1) * a.ldw;
	float acc[NT][4] = {};
	const int nslice = (a.K + 31) / 32;
	constexpr int U = 4; // slices requested before the first is used: 8 x 16 bytes in flight per lane
	if (!a.w_immutable && !waited) pdl_wait_prev(), waited = true;
	for (int s0 = warp; s0 < nslice; s0 += NW * U) {
		uint4 A0[U], A1[U];
#pragma unroll
		for (int u = 0; u < U; ++u) {
			const int k = (s0 + NW * u) * 32 + 8 * t;
			A0[u] = A1[u] = make_uint4(0, 0, 0, 0);
			if (k < a.K) A0[u] = __ldcs((const uint4*)(w0 + k)), A1[u] = __ldcs((const uint4*)(w1 + k));
		}
		if (!waited) pdl_wait_prev(), waited = true; // the first weights (immutable) are already on their way; the activations need the previous kernel
#pragma unroll
		for (int u = 0; u < U; ++u) {
			const int k = (s0 + NW * u) * 32 + 8 * t;
			const uint32_t F0[4] = {A0[u].x, A1[u].x, A0[u].y, A1[u].y}, F1[4] = {A0[u].z, A1[u].z, A0[u].w, A1[u].w};
#pragma unroll
			for (int j = 0; j < NT; ++j) {
				uint4 B = make_uint4(0, 0, 0, 0);
				const int n = j * 8 + g;
				if (n < gr.count && k < a.K) B = *(const uint4*)(X + (size_t)n * a.ldx + k);
				const uint32_t B0[2] = {B.x, B.y}, B1[2] = {B.z, B.w};
				mma_bf16_16816(acc[j], F0, B0);
				mma_bf16_16816(acc[j], F1, B1);
			}
		}
	}
	if (!waited) pdl_wait_prev(); // a warp without a slice still must not write before the previous kernel is done
#pragma unroll
	for (int j = 0; j < NT; ++j) {
		red[warp][g][j * 8 + 2 * t] = acc[j][0], red[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
		red[warp][g + 8][j * 8 + 2 * t] = acc[j][2], red[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
	}
	__syncthreads();
	for (int i = tid; i < 16 * NT * 8; i += NW * 32) {
		const int n = i / 16, r = i % 16; // consecutive threads: consecutive weight rows of one token
		float v = 0.f;
#pragma unroll
		for (int w = 0; w < NW; ++w) v += red[w][r][n];
		gemm_store<bf16>(a, z, gr, n, m0 + r, v);
	}
}

// ---------------------------------------------------------------- sampling helper
__global__ void k_seq_argmax(const float* logits, int vocab, int* out) {
	pdl_enter(); // programmatic dependent launch: let the next kernel's launch overlap this one, then wait for the previous one
	__shared__ float bv[32];
	__shared__ int bi[32];
	const float* row = logits + (size_t)blockIdx.x * vocab;
	float v = -INFINITY;
	int ix = 0x7fffffff;
	for (int i = threadIdx.x; i < vocab; i += blockDim.x)
		if (row[i] > v) v = row[i], ix = i; // ascending i per thread: the first maximum stays
	for (int o = 16; o > 0; o >>= 1) {
		const float ov = __shfl_xor_sync(0xffffffffu, v, o);
		const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
		if (ov > v || (ov == v && oi < ix)) v = ov, ix = oi;
	}
	if ((threadIdx.x & 31) == 0) bv[threadIdx.x >> 5] = v, bi[threadIdx.x >> 5] = ix;
	__syncthreads();
	if (threadIdx.x == 0) {
		for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
			if (bv[w] > v || (bv[w] == v && bi[w] < ix)) v = bv[w], ix = bi[w];
		out[blockIdx.x] = ix;
	}
}
