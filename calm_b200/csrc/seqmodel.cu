// seqmodel.cu -- host side of libcalm_b200_seq.so (include/calm_b200_seq.h): the state manager (sequence slots, a paged
// cache shared by every position-indexed cache of the model, per-slot recurrent and convolution state) and the step
// function that runs a packed batch of tokens through the layer list.

#include "../../include/calm_b200_seq.h"

#include <math.h>
#include <string.h>

#include <algorithm>
#include <array>
#include <functional>
#include <map>
#include <type_traits>
#include <vector>

#include "seqkernels.cuh"
#include "seqgemm_tc.cuh"

namespace {

uint64_t g_seq_launches = 0;

enum Kind { KD_EMBED, KD_NORM, KD_GEMM, KD_GEMM_TC, KD_GEMM_SKINNY, KD_CONV, KD_ATTN_LATENT, KD_ATTN_WINDOW, KD_DELTA, KD_ELEMENT, KD_QK, KD_GLA, KD_ROUTE, KD_HYPER, KD_LINPREP, KD_COUNT };
const char* const kKindNames[KD_COUNT] = {"embed", "norm", "gemm", "gemm_tcgen05", "gemm_skinny", "conv", "attention_latent", "attention_window", "delta_scan", "elementwise",
                                          "qk_prep", "gla_scan", "moe_route", "hyper", "lin_prep"};

// what one run of a layer owns (a looped layer has one of these per pass)
struct RunState {
	int layer = 0;
	bool readd = false;      // the embedding output is added to the stream right before this run
	float* cache_a = nullptr; // SEQ_LATENT: latent rows; SEQ_WINDOW / SEQ_GQA: key rows
	float* cache_b = nullptr; // SEQ_WINDOW / SEQ_GQA: value rows
	float* conv = nullptr;    // [slots][taps-1][channels]
	float* delta = nullptr;   // SEQ_DELTA / SEQ_GLA: the recurrent state [slots][heads][dim][vdim]
	size_t conv_per_slot = 0, delta_per_slot = 0;
	float* mstate = nullptr;  // SEQ_MLSTM: the running maximum of the log gates [slots][heads]
	size_t m_per_slot = 0;
	float* slopes = nullptr;  // SEQ_GQA with dist_bias: the penalty per position of distance, per head
	std::vector<RunState> sub; // SEQ_PAIR: the two mixers' own caches and state
};

struct Slot {
	bool open = false;
	int len = 0;
	int last_tok = -1; // the token before the next one (the bigram embedding reads it); -1: the sequence is empty
	std::vector<int> pages;
};

struct Seq {
	SeqModel m;
	std::vector<SeqLayer> layers;
	std::vector<std::array<SeqLayer, 2>> pairs;
	std::vector<RunState> runs;
	std::map<const SeqLayer*, std::pair<double*, float>> rot; // per SEQ_GQA record (a layer's, or one of a pair's): angle step of every rotated pair (device), factor on cos and sin
	cudaStream_t stream = nullptr;
	int sms = 0;
	bool tc = false; // tcgen05 products available (bf16 mode)

	// state manager
	int n_pages = 0, max_pages = 0;
	std::vector<int> free_pages;
	std::vector<Slot> slots;
	std::vector<int> table; // host mirror of the page table
	int* table_dev = nullptr;

	// per-step batch description
	int cap_tokens = 0, cap_seqs = 0, cap_want = 0;
	int *d_tok = nullptr, *d_tslot = nullptr, *d_tpos = nullptr, *d_tfirst = nullptr, *d_tprev = nullptr, *d_sstart = nullptr, *d_scount = nullptr, *d_spos0 = nullptr, *d_sslot = nullptr,
	    *d_want = nullptr, *d_argmax = nullptr;
	std::vector<int> h_meta;

	// workspace for cap_tokens tokens
	float *x = nullptr, *x0 = nullptr, *proj = nullptr, *f[6] = {};
	void* ah = nullptr;                               // parallel blocks: a dense unit's hidden activations, written by the mixer's input product
	size_t w_ah = 0;
	float* mo = nullptr;                              // parallel blocks: the mixer's output until the feed-forward's is added with it; hyper blocks: a sublayer's output
	float* fsh = nullptr;                             // routed feed-forward with a shared unit: the product [shared gate | shared up | router logits]
	size_t w_fsh = 0;
	float* lin = nullptr;                             // scan input of the linear recurrences served by the gated-linear-attention scan: rows [q | k | v]
	size_t w_lin = 0;
	int streams = 1;
	bool h_ready = false;                             // hyper blocks: hA already holds the next sublayer's normed input (the last write formed it)
	// routed experts: choices and weights per token, groups, and the grouped activations of max_top choices per token
	int max_top = 0, max_experts = 0;
	size_t w_moe_ff = 0;
	int *moe_sel = nullptr, *moe_perm = nullptr, *moe_inv = nullptr, *moe_seg = nullptr;
	float *moe_wt = nullptr, *moe_y = nullptr, *moe_d = nullptr;
	void *moe_x = nullptr, *moe_a = nullptr;
	void *hA = nullptr, *a1 = nullptr, *a2 = nullptr; // activation type (float or bf16)
	size_t w_proj = 0, w_f = 0, w_a = 0;              // widths (elements per token)
	// prompt attention as products: gathered keys / transposed values of one key head, scores and probabilities
	bool attn_products = true;
	bf16 *att_kb = nullptr, *att_vt = nullptr, *att_p = nullptr;
	float* att_s = nullptr;
	size_t cap_kb = 0, cap_vt = 0, cap_sp = 0;
	void* a3 = nullptr;                               // queries in the activation type
	std::vector<int> hb_start, hb_count, hb_pos0, hb_slot; // host copy of the batch description
	int* d_skip = nullptr;                            // [N] 1: token served by the product path
	int n_on_products = 0, tok_on_products = 0;       // sequences / tokens of this step on the product path
	float* part = nullptr; // partial attention results of key-split launches
	size_t part_cap = 0;
	float* logits = nullptr;
	void* hW = nullptr; // normed rows of the wanted tokens
	int last_want = 0, last_tokens = 0;

	bool trace = false;
	float* trace_buf = nullptr;
	int trace_cap = 0;

	// decode steps (one token per sequence) replay a captured graph per (batch, wanted rows, key shares of every attention run)
	bool use_graph = true;
	bool pdl = true;
	std::map<std::vector<int>, std::pair<cudaGraphExec_t, int>> graphs; // -> (graph, launches in it)

	bool perf = false;
	double kind_ms[KD_COUNT] = {}, kind_bytes[KD_COUNT] = {}, kind_flops[KD_COUNT] = {};
	long kind_launches[KD_COUNT] = {};
	cudaEvent_t ev[2] = {nullptr, nullptr}, timer[2] = {nullptr, nullptr};
};

void* dalloc(size_t bytes) {
	void* p = nullptr;
	CUDA_CHECK(cudaMalloc(&p, bytes ? bytes : 16));
	return p;
}
int cdiv(long a, long b) { return (int)((a + b - 1) / b); }
size_t act_size(const Seq& s) { return s.m.exact ? sizeof(float) : sizeof(bf16); }

// every launch goes through here: counts it and, while profiling, brackets it with events
template <typename F>
void run_kernel(Seq& s, int kind, double bytes, double flops, F&& launch) {
	if (s.perf) CUDA_CHECK(cudaEventRecord(s.ev[0], s.stream));
	launch();
	CUDA_CHECK(cudaGetLastError());
	++g_seq_launches;
	if (s.perf) {
		CUDA_CHECK(cudaEventRecord(s.ev[1], s.stream));
		CUDA_CHECK(cudaEventSynchronize(s.ev[1]));
		float ms = 0;
		CUDA_CHECK(cudaEventElapsedTime(&ms, s.ev[0], s.ev[1]));
		s.kind_ms[kind] += ms, s.kind_bytes[kind] += bytes, s.kind_flops[kind] += flops, ++s.kind_launches[kind];
	}
}

// Every kernel goes out with programmatic stream serialization allowed: it may be launched while its predecessor still runs and
// parks in pdl_enter() until that one has completed and flushed (a no-op attribute-less launch when CALM_B200_SEQ_PDL=0).
template <typename... KArgs, typename... Args>
void launch_k(Seq& s, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s.stream;
	cudaLaunchAttribute at[1];
	at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
	at[0].val.programmaticStreamSerializationAllowed = 1;
	cfg.attrs = at, cfg.numAttrs = s.pdl ? 1 : 0;
	CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
}

size_t in_rows(const SeqLayer& L) {
	switch (L.type) {
	case SEQ_LATENT: return (size_t)L.q_rank + L.kv_rank + L.heads;
	case SEQ_DELTA: return (size_t)2 * L.kv_heads * L.dim + (size_t)L.heads * L.vdim + L.heads + L.a_rank + L.g_rank;
	case SEQ_GQA: return (size_t)L.heads * L.dim + (size_t)L.kv_heads * L.dim + (size_t)L.kv_heads * L.vdim + (L.no_gate ? 0 : L.gate_per_head ? (size_t)L.heads : (size_t)L.heads * L.vdim);
	case SEQ_MLSTM: return (size_t)2 * L.heads * L.dim + (size_t)2 * L.heads * L.vdim + 2 * L.heads;
	case SEQ_HGRN2: return (size_t)2 * L.heads * L.dim + (size_t)L.heads * L.vdim;
	case SEQ_MAMBA2: return (size_t)2 * L.heads * L.vdim + (size_t)2 * L.kv_heads * L.dim + L.heads;
	case SEQ_PAIR: return 0;
	case SEQ_GLA: return (size_t)2 * L.heads * L.dim + (size_t)2 * L.heads * L.vdim + L.a_rank;
	default: return (size_t)L.heads * L.dim + (size_t)L.kv_heads * L.dim + (size_t)L.kv_heads * L.vdim;
	}
}
// row stride of the input projection's fp32 output: the mixer's rows, and a router's that ride along (rounded to whole float4s)
int proj_stride(const SeqLayer& L) {
	if (L.in_tail <= 0) return (int)in_rows(L);
	return (int)((in_rows(L) + (L.ff_kind == SEQ_FF_MOE ? L.in_tail : 0) + 3) & ~(size_t)3);
}
// a pair whose own record carries the stacked input matrix: column of the second mixer's first row, and the row stride of the fp32 product
// (a gated-linear-attention in second place keeps its decay input out of it)
int pair_offset(const SeqLayer& L) { return (int)((in_rows(L.pair[0]) + 7) & ~(size_t)7); }
int pair_stride(const SeqLayer& L) {
	const size_t m = pair_offset(L) + in_rows(L.pair[1]) - (L.pair[1].type == SEQ_GLA ? L.pair[1].a_rank : 0);
	return (int)((m + 3) & ~(size_t)3);
}
int conv_channels(const SeqLayer& L) {
	if (L.type == SEQ_DELTA) return 2 * L.kv_heads * L.dim + L.heads * L.vdim;
	if (L.type == SEQ_WINDOW) return L.heads * L.dim + L.kv_heads * L.dim + L.kv_heads * L.vdim;
	if (L.type == SEQ_MAMBA2) return L.heads * L.vdim + 2 * L.kv_heads * L.dim;
	return 0;
}
// value columns of a linear recurrence's scan: the mLSTM carries its normaliser as one more column; whole float4s either way
int lin_vs(const SeqLayer& L) { return ((L.type == SEQ_MLSTM ? L.vdim + 1 : L.vdim) + 3) & ~3; }
bool is_lin(const SeqLayer& L) { return L.type == SEQ_MLSTM || L.type == SEQ_HGRN2 || L.type == SEQ_MAMBA2; }
// gated linear attention: key channels per lane when `lanes` lanes share a value column, the scan's shared memory, the row length
// of a value column in the state (the same whichever lane count a step runs with), and the kernel's instantiations
int gla_rows(int dim, int lanes) {
	const int rows = cdiv(dim, lanes);
	for (int r : {4, 8, 16, 24, 32, 64})
		if (rows <= r && (r != 24 || lanes == 4) && (r != 4 || lanes != 4)) return r; // the instantiations of gla_each
	return 64;
}
size_t gla_smem(int R, int lanes) { return ((size_t)2 * GLA_TB * (3 * lanes * (R + 4) + 128 / lanes) + 2 * GLA_TB * (128 / lanes)) * sizeof(float); }
int gla_ldstate(int dim) { return std::max({4 * gla_rows(dim, 4), 8 * gla_rows(dim, 8), 16 * gla_rows(dim, 16)}); }
template <typename F>
void gla_each(F&& f) {
	auto one = [&](auto r, auto p) { f(r, p); };
	one(std::integral_constant<int, 8>{}, std::integral_constant<int, 4>{}), one(std::integral_constant<int, 16>{}, std::integral_constant<int, 4>{});
	one(std::integral_constant<int, 24>{}, std::integral_constant<int, 4>{}), one(std::integral_constant<int, 32>{}, std::integral_constant<int, 4>{});
	one(std::integral_constant<int, 64>{}, std::integral_constant<int, 4>{});
	one(std::integral_constant<int, 4>{}, std::integral_constant<int, 8>{}), one(std::integral_constant<int, 8>{}, std::integral_constant<int, 8>{});
	one(std::integral_constant<int, 16>{}, std::integral_constant<int, 8>{}), one(std::integral_constant<int, 32>{}, std::integral_constant<int, 8>{});
	one(std::integral_constant<int, 4>{}, std::integral_constant<int, 16>{}), one(std::integral_constant<int, 8>{}, std::integral_constant<int, 16>{});
	one(std::integral_constant<int, 16>{}, std::integral_constant<int, 16>{});
}
// query heads per CTA of the attention kernel: divides the group, keeps the accumulators in registers and the queries in shared memory
int attn_tile(int group, int kd, int vd) {
	if (vd > 2 * ATT_THREADS) return 1; // wide values: one head per CTA
	int t = group;
	while (t > 1 && ((size_t)t * (kd + ATT_KC + 3) * sizeof(float) > 96 * 1024 || t > 16)) {
		int d = t - 1;
		while (group % d) --d;
		t = d;
	}
	return t;
}
size_t attn_smem(int tile, int kd) { return ((size_t)tile * (kd + ATT_KC + 3) + 4) * sizeof(float); }

void validate_mixer(const Seq& s, int i, const SeqLayer& L, bool inner) {
	const SeqModel& m = s.m;
	{
		if (L.type == SEQ_PAIR) {
			if (inner || !L.pair) CALM_FATAL("seq: layer %d: a pair holds two plain mixers", i);
			validate_mixer(s, i, L.pair[0], true), validate_mixer(s, i, L.pair[1], true);
			if (L.w_in)
				for (int k = 0; k < 2; ++k)
					if ((L.pair[k].type != SEQ_GQA && L.pair[k].type != SEQ_GLA) || L.pair[k].w_in || L.pair[k].in_tail)
						CALM_FATAL("seq: layer %d: a pair with a stacked input matrix holds grouped-query and gated linear attention, without input matrices of their own", i);
			return;
		}
		if (L.heads < 1 || L.dim < 1 || L.vdim < 1) CALM_FATAL("seq: layer %d: heads, dim and vdim must be positive", i);
		if (is_lin(L)) {
			if (L.dim > 256) CALM_FATAL("seq: layer %d: a linear-recurrence head holds at most 256 key channels", i);
			if (L.type == SEQ_MLSTM && !(L.gate_cap > 0.f)) CALM_FATAL("seq: layer %d: gate_cap must be positive", i);
			if (L.type == SEQ_MAMBA2) {
				if (L.kv_heads < 1 || L.heads % L.kv_heads) CALM_FATAL("seq: layer %d: heads must be a multiple of the groups", i);
				if (L.norm_groups < 1 || (L.heads * L.vdim) % L.norm_groups) CALM_FATAL("seq: layer %d: norm_groups must divide heads * vdim", i);
				if (L.taps < 1) CALM_FATAL("seq: layer %d: taps must be positive", i);
			}
		} else if (L.type == SEQ_LATENT) {
			if (L.q_rank < 1 || L.kv_rank < 1) CALM_FATAL("seq: layer %d: latent ranks must be positive", i);
			if (cdiv(L.kv_rank, ATT_THREADS) > ATT_MAXI) CALM_FATAL("seq: layer %d: kv_rank %d is more than the attention kernel holds", i, L.kv_rank);
		} else if (L.type == SEQ_DELTA || L.type == SEQ_WINDOW) {
			if (L.kv_heads < 1 || L.heads % L.kv_heads) CALM_FATAL("seq: layer %d: heads must be a multiple of kv_heads", i);
			if (L.taps < 1) CALM_FATAL("seq: layer %d: taps must be positive", i);
			if (L.type == SEQ_DELTA) {
				if (L.vdim > 1024) CALM_FATAL("seq: layer %d: vdim above 1024", i);
				if (((size_t)L.dim * L.vdim + 3 * (size_t)L.dim) * sizeof(float) > 227 * 1024) CALM_FATAL("seq: layer %d: a %d x %d state does not fit shared memory", i, L.dim, L.vdim);
				if (L.a_rank < 1 || L.g_rank < 1) CALM_FATAL("seq: layer %d: decay and gate ranks must be positive", i);
			} else if (cdiv(L.vdim, ATT_THREADS) > ATT_MAXI) CALM_FATAL("seq: layer %d: vdim too large", i);
		} else if (L.type == SEQ_GQA) {
			if (L.kv_heads < 1 || L.heads % L.kv_heads) CALM_FATAL("seq: layer %d: heads must be a multiple of kv_heads", i);
			if (cdiv(L.vdim, ATT_THREADS) > ATT_MAXI) CALM_FATAL("seq: layer %d: vdim too large", i);
			if (L.rot_dims < 0 || L.rot_dims > L.dim || L.rot_dims % 2) CALM_FATAL("seq: layer %d: rot_dims must be even and at most dim", i);
			if (L.rot_dims > 0 && !(L.rot_base > 0.f)) CALM_FATAL("seq: layer %d: rot_base must be positive", i);
			if ((L.q_norm == nullptr) != (L.k_norm == nullptr)) CALM_FATAL("seq: layer %d: query and key norm come together", i);
			if (L.keep_first < 0) CALM_FATAL("seq: layer %d: keep_first is negative", i);
		} else if (L.type == SEQ_GLA) {
			if (L.dim > 256) CALM_FATAL("seq: layer %d: a gated-linear-attention head holds at most 256 key channels", i);
			if (L.a_rank < 1) CALM_FATAL("seq: layer %d: the decay rank must be positive", i);
			if (!(L.tau > 0.f)) CALM_FATAL("seq: layer %d: tau must be positive", i);
		} else CALM_FATAL("seq: layer %d: unknown mixer %d", i, L.type);
		if ((L.type != SEQ_GQA && (L.chunk || L.dist_bias || L.add_one || L.v_norm || L.no_gate || L.qk_per_head || L.gate_per_head || L.scores_f32)) || L.chunk < 0)
			CALM_FATAL("seq: layer %d: chunk, dist_bias, add_one, v_norm, no_gate, qk_per_head, gate_per_head and scores_f32 are options of SEQ_GQA", i);
		(void)m;
	}
}

void validate(const Seq& s) {
	const SeqModel& m = s.m;
	if (m.vocab < 1 || m.width < 1 || m.n_layers < 1) CALM_FATAL("seq: empty model");
	if (m.page < 1 || m.max_seqs < 1 || m.max_tokens < 1) CALM_FATAL("seq: page, max_seqs and max_tokens must be positive");
	if (m.loop_times > 1 && !(0 <= m.loop_start && m.loop_start < m.loop_stop && m.loop_stop <= m.n_layers)) CALM_FATAL("seq: bad loop span");
	if (m.streams < 0 || m.streams > HC_MAX) CALM_FATAL("seq: at most %d streams", HC_MAX);
	if (m.block != SEQ_BLOCK_HYPER && m.streams > 1) CALM_FATAL("seq: several streams need hyper blocks");
	if (m.block == SEQ_BLOCK_HYPER && m.loop_times > 1) CALM_FATAL("seq: hyper blocks are not served inside a looped span");
	if (m.pos_table && m.max_positions < 1) CALM_FATAL("seq: a position table needs max_positions");
	for (int i = 0; i < m.n_layers; ++i) {
		const SeqLayer& L = s.layers[i];
		validate_mixer(s, i, L, false);
		if (m.block == SEQ_BLOCK_HYPER && (!L.hc1.in || !L.hc1.out || !L.hc1.mix || (L.ff > 0 && (!L.hc2.in || !L.hc2.out || !L.hc2.mix))))
			CALM_FATAL("seq: layer %d: hyper blocks need in, out and mix of every sublayer", i);
		if (m.block != SEQ_BLOCK_HYPER && m.block != SEQ_BLOCK_POST && (L.type == SEQ_PAIR || is_lin(L))) CALM_FATAL("seq: layer %d: this mixer is served in hyper and post-norm blocks", i);
		if (L.ff > 0) {
			if (L.ff_kind < SEQ_FF_CLAMPED || L.ff_kind > SEQ_FF_GATED) CALM_FATAL("seq: layer %d: unknown feed-forward kind %d", i, L.ff_kind);
			if (L.ff_kind == SEQ_FF_GATED && L.ff_act != SEQ_ACT_SILU && L.ff_act != SEQ_ACT_GELU_TANH) CALM_FATAL("seq: layer %d: unknown activation %d", i, L.ff_act);
			if (L.in_tail != 0 && (m.block != SEQ_BLOCK_PARALLEL || L.in_tail != (L.ff_kind == SEQ_FF_MOE ? L.experts : L.ff_kind == SEQ_FF_RELU2 ? L.ff : -1)))
				CALM_FATAL("seq: layer %d: in_tail must be the router's or the up projection's row count, in a parallel block", i);
			if (L.ff_kind == SEQ_FF_MOE) {
				if (L.experts < 1 || L.top < 1 || L.top > L.experts + L.ident) CALM_FATAL("seq: layer %d: 1 <= top <= experts", i);
				if (m.block == SEQ_BLOCK_SERIAL) CALM_FATAL("seq: layer %d: routed experts are not served in serial blocks", i);
				if (L.ident < 0 || L.top > L.experts + L.ident || L.shared_ff < 0) CALM_FATAL("seq: layer %d: bad identity experts or shared unit", i);
				if (!L.w_router && L.in_tail == 0 && L.shared_ff == 0) CALM_FATAL("seq: layer %d: the router's rows ride either behind the shared unit's or in w_router", i);
				if (m.block != SEQ_BLOCK_HYPER && (L.ident || L.route_mode == 1)) CALM_FATAL("seq: layer %d: identity experts and route_mode 1 are served in hyper blocks", i);
				if (m.block != SEQ_BLOCK_HYPER && m.block != SEQ_BLOCK_POST && L.shared_ff) CALM_FATAL("seq: layer %d: the shared unit is served in hyper and post-norm blocks", i);
				if (L.route_mode < 0 || L.route_mode > 2) CALM_FATAL("seq: layer %d: unknown route_mode %d", i, L.route_mode);
				if (m.block != SEQ_BLOCK_POST && (L.expert_act || L.weight_input || L.shared_gate)) CALM_FATAL("seq: layer %d: relu^2 experts, weights on the input and the gated shared unit are served in post-norm blocks", i);
				if (m.block == SEQ_BLOCK_POST && L.shared_ff && !L.expert_act) CALM_FATAL("seq: layer %d: post-norm blocks serve the shared unit in the relu^2 form", i);
				if (L.weight_input && !L.expert_act) CALM_FATAL("seq: layer %d: a weight on the input is served for relu^2 experts", i);
				if (L.shared_gate && !L.shared_ff) CALM_FATAL("seq: layer %d: a shared gate needs a shared unit", i);
			}
		}
	}
	if (m.norm_kind != SEQ_NORM_DYT && m.norm_kind != SEQ_NORM_RMS) CALM_FATAL("seq: unknown norm kind %d", m.norm_kind);
	if (m.block < SEQ_BLOCK_SERIAL || m.block > SEQ_BLOCK_POST) CALM_FATAL("seq: unknown block form %d", m.block);
	if (m.block == SEQ_BLOCK_POST && (m.norm_kind != SEQ_NORM_RMS || m.norm_scalar || m.loop_times > 1)) CALM_FATAL("seq: post-norm blocks use the RMS norm with a weight per column, outside looped spans");
	if (m.bigram && (m.bigram_buckets < 1 || m.bigram_mul_prev < 0 || m.bigram_mul_cur < 0)) CALM_FATAL("seq: a bigram table needs buckets >= 1 and multipliers >= 0");
	if (m.block == SEQ_BLOCK_HYPER && m.norm_kind != SEQ_NORM_RMS) CALM_FATAL("seq: hyper blocks use the RMS norm");
	if (m.block == SEQ_BLOCK_SERIAL && m.norm_kind != SEQ_NORM_DYT)
		CALM_FATAL("seq: serial blocks fold their second norm into the product before it, which only a norm without row statistics (Dynamic Tanh) allows");
}

void drop_graphs(Seq& s) {
	for (auto& kv : s.graphs) cudaGraphExecDestroy(kv.second.first);
	s.graphs.clear();
}

void reserve_tokens(Seq& s, int N, int B, int W) {
	if (B > s.cap_seqs || N > s.cap_tokens || W > s.cap_want) drop_graphs(s); // captured launches hold the old addresses
	if (B > s.cap_seqs || N > s.cap_tokens) {
		const int cn = std::max(N, s.cap_tokens), cb = std::max(B, s.cap_seqs);
		CUDA_CHECK(cudaStreamSynchronize(s.stream));
		cudaFree(s.d_tok);
		s.d_tok = (int*)dalloc(((size_t)6 * cn + 4 * cb) * sizeof(int));
		s.d_tslot = s.d_tok + cn, s.d_tpos = s.d_tslot + cn, s.d_tfirst = s.d_tpos + cn, s.d_skip = s.d_tfirst + cn, s.d_tprev = s.d_skip + cn;
		s.d_sstart = s.d_tprev + cn, s.d_scount = s.d_sstart + cb, s.d_spos0 = s.d_scount + cb, s.d_sslot = s.d_spos0 + cb;
		s.cap_seqs = cb;
	}
	if (W > s.cap_want) {
		CUDA_CHECK(cudaStreamSynchronize(s.stream));
		cudaFree(s.d_want), cudaFree(s.d_argmax), cudaFree(s.logits), cudaFree(s.hW);
		s.cap_want = std::max(W, 2 * s.cap_want);
		s.d_want = (int*)dalloc(s.cap_want * sizeof(int));
		s.d_argmax = (int*)dalloc(s.cap_want * sizeof(int));
		s.logits = (float*)dalloc((size_t)s.cap_want * s.m.vocab * sizeof(float));
		s.hW = dalloc((size_t)s.cap_want * s.m.width * act_size(s));
	}
	if (N > s.cap_tokens) {
		const size_t cn = N;
		cudaFree(s.x), cudaFree(s.x0), cudaFree(s.proj), cudaFree(s.hA), cudaFree(s.a1), cudaFree(s.a2), cudaFree(s.a3), cudaFree(s.mo);
		for (float*& p : s.f) cudaFree(p);
		if (s.m.block != SEQ_BLOCK_SERIAL) s.mo = (float*)dalloc(cn * s.m.width * sizeof(float));
		if (s.w_lin) cudaFree(s.lin), s.lin = (float*)dalloc(cn * s.w_lin * sizeof(float));
		if (s.w_fsh) cudaFree(s.fsh), s.fsh = (float*)dalloc(cn * s.w_fsh * sizeof(float));
		if (s.w_ah) cudaFree(s.ah), s.ah = dalloc(cn * s.w_ah * act_size(s));
		if (s.max_top > 0) {
			cudaFree(s.moe_sel), cudaFree(s.moe_wt), cudaFree(s.moe_y), cudaFree(s.moe_d), cudaFree(s.moe_x), cudaFree(s.moe_a);
			const size_t pairs = cn * s.max_top;
			s.moe_sel = (int*)dalloc((3 * pairs + s.max_experts + 1) * sizeof(int));
			s.moe_perm = s.moe_sel + pairs, s.moe_inv = s.moe_perm + pairs, s.moe_seg = s.moe_inv + pairs;
			s.moe_wt = (float*)dalloc(pairs * sizeof(float));
			s.moe_y = (float*)dalloc(pairs * 2 * s.w_moe_ff * sizeof(float));
			s.moe_d = (float*)dalloc(pairs * s.m.width * sizeof(float));
			s.moe_x = dalloc(pairs * s.m.width * act_size(s));
			s.moe_a = dalloc(pairs * s.w_moe_ff * act_size(s));
		}
		s.x = (float*)dalloc(cn * s.streams * s.m.width * sizeof(float));
		s.x0 = (float*)dalloc(cn * s.m.width * sizeof(float));
		s.proj = (float*)dalloc(cn * s.w_proj * sizeof(float));
		for (float*& p : s.f) p = (float*)dalloc(cn * s.w_f * sizeof(float));
		s.hA = dalloc(cn * s.m.width * act_size(s));
		s.a1 = dalloc(cn * s.w_a * act_size(s));
		s.a2 = dalloc(cn * s.w_a * act_size(s));
		s.a3 = dalloc(cn * s.w_a * act_size(s));
		s.cap_tokens = N;
	}
	if (s.trace && (size_t)N * s.runs.size() > (size_t)s.trace_cap) {
		cudaFree(s.trace_buf);
		s.trace_cap = N * (int)s.runs.size();
		s.trace_buf = (float*)dalloc((size_t)s.trace_cap * s.m.width * sizeof(float));
	}
}

// ---------------------------------------------------------------- launches

// what a product's epilogue may take besides the accumulator
struct GemmExtra {
	const void* bias = nullptr;  // bf16 [batch][M]
	const float* res = nullptr;  // EPI_RES: second addend
	const float* gate = nullptr; // EPI_ACT: sigmoid gate
	long ldgate = 0, gbs = 0;
	const int* seg = nullptr;    // grouped product: rows of batch z
	int x_rows = 0;              // grouped product: rows of X / Y over all groups
	float epi_f = 0.f;           // EPI_DECAY: exponent
	float out_scale = 0.f;       // != 0: factor on the accumulator
	int split = 0;               // columns from here on leave in the activation type to Y2: as relu(.)^2, or unchanged when split_act is 1
	int split_act = 0;
	void* Y2 = nullptr;
	long ldy2 = 0;
	const float* rs = nullptr;   // a factor per row on the accumulator: rs[(rs_idx ? rs_idx[row] : row) * rs_ld], through a sigmoid when rs_act
	const int* rs_idx = nullptr;
	long rs_ld = 1;
	int rs_act = 0;
};
void gemm(Seq& s, const void* X, long ldx, long xbs, const void* W, long ldw, long wbs, void* Y, long ldy, long ybs, int N, int M, int K, int batch, int epi,
          const SeqNorm* nrm = nullptr, int kind_as = -1, bool w_immutable = true, const GemmExtra* ex = nullptr) {
	GemmArgs a;
	const GemmExtra none;
	if (!ex) ex = &none;
	a.bias = (const bf16*)ex->bias, a.res = ex->res, a.gate = ex->gate, a.ldgate = ex->ldgate, a.gbs = ex->gbs, a.seg = ex->seg, a.x_rows = ex->x_rows, a.epi_f = ex->epi_f, a.split = ex->split, a.split_act = ex->split_act, a.Y2 = ex->Y2, a.ldy2 = ex->ldy2, a.out_scale = ex->out_scale;
	a.rs = ex->rs, a.rs_idx = ex->rs_idx, a.rs_ld = ex->rs_ld, a.rs_act = ex->rs_act;
	a.w_immutable = w_immutable;
	a.X = X, a.ldx = ldx, a.xbs = xbs, a.W = (const bf16*)W, a.ldw = ldw, a.wbs = wbs, a.Y = Y, a.ldy = ldy, a.ybs = ybs;
	a.N = N, a.M = M, a.K = K, a.epi = epi;
	a.nw = nrm ? (const bf16*)nrm->w : nullptr, a.nb = nrm ? (const bf16*)nrm->b : nullptr, a.na = nrm ? (const bf16*)nrm->alpha : nullptr;
	// a grouped product does the work of its x_rows rows, and reads at most that many groups' weights
	const double rows = ex->seg ? (double)ex->x_rows : (double)N * batch, mats = ex->seg ? std::min((double)batch, rows) : (double)batch;
	const double flops = 2.0 * rows * M * K;
	const double bytes = mats * M * K * 2 + rows * K * act_size(s) + rows * M * 4;
	if (s.tc && gemm_tc_fits(a, batch)) {
		bool launched = false;
		run_kernel(s, kind_as >= 0 ? kind_as : KD_GEMM_TC, bytes, flops, [&] { launched = gemm_tc_launch(a, batch, s.stream); });
		if (launched) return;
	}
	auto al8 = [](long v) { return v % 8 == 0; };
	if (!s.m.exact && N <= 32 && K % 8 == 0 && al8(ldx) && al8(ldw) && al8(xbs) && al8(wbs) && ((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0) {
		const dim3 grid(cdiv(M, 16), 1, batch);
		const bool few = (long)cdiv(M, 16) * batch < 3L * s.sms && K >= 1024; // few CTAs: twice the warps per CTA keep as many bytes in flight
		run_kernel(s, kind_as >= 0 ? kind_as : KD_GEMM_SKINNY, bytes, flops, [&] {
			if (few) {
				if (N <= 8) launch_k(s, k_seq_gemm_skinny<1, 16>, grid, 512, 0, a);
				else if (N <= 16) launch_k(s, k_seq_gemm_skinny<2, 16>, grid, 512, 0, a);
				else launch_k(s, k_seq_gemm_skinny<4, 16>, grid, 512, 0, a);
			} else {
				if (N <= 8) launch_k(s, k_seq_gemm_skinny<1, 8>, grid, 256, 0, a);
				else if (N <= 16) launch_k(s, k_seq_gemm_skinny<2, 8>, grid, 256, 0, a);
				else launch_k(s, k_seq_gemm_skinny<4, 8>, grid, 256, 0, a);
			}
		});
		return;
	}
	const dim3 grid(cdiv(M, 64), cdiv(N, 64), batch);
	run_kernel(s, kind_as >= 0 ? kind_as : KD_GEMM, bytes, flops, [&] {
		if (s.m.exact) launch_k(s, k_seq_gemm_f32, grid, 256, 0, a);
		else launch_k(s, k_seq_gemm_bf16, grid, 128, 0, a);
	});
}

void dyt(Seq& s, void* out, const float* x, const int* rows, const SeqNorm& nm, int R);
// the model's norm on whole rows of the residual stream
void norm(Seq& s, void* out, const float* x, const int* rows, const SeqNorm& nm, int R) {
	if (s.m.norm_kind == SEQ_NORM_DYT) return dyt(s, out, x, rows, nm, R);
	const int W = s.m.width;
	run_kernel(s, KD_NORM, (double)R * W * (4 + act_size(s)), 0, [&] {
		const int threads = std::min(256, std::max(32, cdiv(W, 4 * 32) * 32)); // about four columns per thread, whole warps
		if (s.m.exact) launch_k(s, k_seq_rms<float>, R, threads, 0, (float*)out, x, rows, (const bf16*)nm.w, s.m.norm_offset, s.m.eps, R, W);
		else launch_k(s, k_seq_rms<bf16>, R, threads, 0, (bf16*)out, x, rows, (const bf16*)nm.w, s.m.norm_offset, s.m.eps, R, W);
	});
}
void dyt(Seq& s, void* out, const float* x, const int* rows, const SeqNorm& nm, int R) {
	const size_t n = (size_t)R * s.m.width;
	run_kernel(s, KD_NORM, n * (4 + act_size(s)), 0, [&] {
		if (s.m.exact) launch_k(s, k_seq_dyt<float>, cdiv(n, 256), 256, 0, (float*)out, x, rows, (const bf16*)nm.w, (const bf16*)nm.b, (const bf16*)nm.alpha, R, s.m.width);
		else launch_k(s, k_seq_dyt<bf16>, cdiv(n, 256), 256, 0, (bf16*)out, x, rows, (const bf16*)nm.w, (const bf16*)nm.b, (const bf16*)nm.alpha, R, s.m.width);
	});
}

// most keys a query of this attention sees (0: all earlier positions)
int attn_span(const SeqLayer& L) {
	if (L.type == SEQ_LATENT) return 0;
	int span = L.window > 0 ? L.window + (L.type == SEQ_GQA ? L.keep_first : 0) : 0;
	if (L.type == SEQ_GQA && L.chunk > 0) span = span > 0 ? std::min(span, L.chunk) : L.chunk;
	return span;
}
// hyper blocks: the weighted sum of the streams (in == null: their plain sum) under the model's RMS norm
void hc_read(Seq& s, void* out, const int* rows, const void* in, const SeqNorm& nm, int R) {
	const int W = s.m.width, S = s.streams, wl = s.m.norm_scalar ? 1 : W;
	run_kernel(s, KD_HYPER, (double)R * W * (4.0 * S + act_size(s)), 0, [&] {
		const int threads = std::min(256, std::max(32, cdiv(W, 4 * 32) * 32));
		if (s.m.exact) launch_k(s, k_seq_hc_read<float>, R, threads, 0, (float*)out, s.x, rows, (const bf16*)in, (const bf16*)nm.w, wl, s.m.norm_offset, s.m.eps, R, W, S);
		else launch_k(s, k_seq_hc_read<bf16>, R, threads, 0, (bf16*)out, s.x, rows, (const bf16*)in, (const bf16*)nm.w, wl, s.m.norm_offset, s.m.eps, R, W, S);
	});
}
// CTAs that share the keys of one (token, head tile): few tokens over a long context
int attn_nsplit(const Seq& s, int live_tokens, int tiles, int window, int longest) {
	const int ctas = live_tokens * tiles, chunks = cdiv(window > 0 ? std::min(longest, window) : longest, ATT_KC);
	return ctas >= 2 * s.sms ? 1 : std::max(1, std::min({chunks, 2 * s.sms / ctas, 128}));
}
void ensure_part(Seq& s, size_t need) {
	if (need <= s.part_cap) return;
	CUDA_CHECK(cudaStreamSynchronize(s.stream));
	drop_graphs(s);
	cudaFree(s.part);
	s.part = (float*)dalloc(need * sizeof(float)), s.part_cap = need;
}

// Sequences that bring at least this many tokens to a step have their attention computed as products (bf16 mode).
const int kAttnGemmMin = 16;

void reserve_attn(Seq& s, size_t kb, size_t vt, size_t sp) {
	if (kb <= s.cap_kb && vt <= s.cap_vt && sp <= s.cap_sp) return;
	CUDA_CHECK(cudaStreamSynchronize(s.stream));
	if (kb > s.cap_kb) cudaFree(s.att_kb), s.att_kb = (bf16*)dalloc(kb * sizeof(bf16)), s.cap_kb = kb;
	if (vt > s.cap_vt) cudaFree(s.att_vt), s.att_vt = (bf16*)dalloc(vt * sizeof(bf16)), s.cap_vt = vt;
	if (sp > s.cap_sp) {
		cudaFree(s.att_s), cudaFree(s.att_p);
		s.att_s = (float*)dalloc(sp * sizeof(float)), s.att_p = (bf16*)dalloc(sp * sizeof(bf16)), s.cap_sp = sp;
	}
}

// one sequence's new tokens [first, first + count) at positions pos0.., in blocks of queries that keep S within budget
void attention_products(Seq& s, int kind, const AttArgs& a, bf16* out, const SeqBatch& sb, int slot, int first, int count, int pos0) {
	const int G = a.heads / a.group;
	const size_t budget = (size_t)96 << 20; // elements of S per launch
	for (int t0 = 0; t0 < count;) {
		const int q0 = pos0 + t0;
		int Tb = count - t0;
		// a block of queries ends where a block of positions does; about a thousand queries per launch keep the launches few (what a row
		// does not see of the other blocks is masked, and costs less than more launches would)
		if (a.chunk > 0) Tb = std::min(Tb, (q0 / a.chunk + std::max(1, 1024 / a.chunk)) * a.chunk - q0);
		while (Tb > 64 && (size_t)a.group * Tb * (size_t)(q0 + Tb) > budget) Tb = (Tb + 1) / 2;
		// gathered keys: the kept first positions the block's window has left behind, then everything from the first query's window on
		int k0 = a.window > 0 ? std::max(0, q0 - a.window + 1) : 0;
		if (a.chunk > 0) k0 = std::max(k0, q0 / a.chunk * a.chunk); // the first query's block; later rows mask what lies before theirs
		const int kfb = a.window > 0 ? std::min(a.keep_first, k0) : 0;
		const int C = kfb + q0 + Tb - k0, Cp = (C + 7) & ~7;
		// split: queries [hi | hi | lo] against keys [hi | lo | hi] (depth 3 kd), probabilities [hi | lo] against the values held twice (depth Cp + C)
		const int sx = a.split ? 3 : 1, px = a.split ? 2 : 1;
		reserve_attn(s, (size_t)C * a.kd * sx, (size_t)a.vd * Cp * px, (size_t)a.group * Tb * Cp * px);
		for (int kvh = 0; kvh < G; ++kvh) {
			AttGather g;
			g.kc = a.kc, g.vc = a.vc, g.kld = a.kld, g.vld = a.vld, g.kcol = kvh * a.kd, g.vcol = kvh * a.vd, g.kd = a.kd, g.vd = a.vd;
			g.Kb = s.att_kb, g.Vt = s.att_vt, g.slot = slot, g.k0 = k0, g.C = C, g.Cp = Cp, g.kfb = kfb, g.split = a.split;
			run_kernel(s, kind, (double)C * (a.kd + a.vd) * (4 + 2 * sx), 0, [&] { launch_k(s, k_seq_attn_gather, dim3(cdiv(Cp, 32), 4), 256, 0, g, sb); });
			const int h0 = kvh * a.group;
			const bf16* q = (const bf16*)s.a3 + ((size_t)(first + t0) * a.heads + h0) * a.kd * sx;
			gemm(s, q, (long)a.heads * a.kd * sx, a.kd * sx, s.att_kb, a.kd * sx, 0, s.att_s, Cp, (long)Tb * Cp, Tb, C, a.kd * sx, a.group, EPI_F32, nullptr, kind, false);
			AttSoftmax sm;
			sm.S = s.att_s, sm.P = s.att_p, sm.T = Tb, sm.C = C, sm.Cp = Cp, sm.qpos0 = q0, sm.k0 = k0, sm.window = a.window, sm.scale = a.scale;
			sm.keep_first = a.window > 0 ? a.keep_first : 0, sm.kfb = kfb, sm.split = a.split;
			sm.chunk = a.chunk, sm.slopes = a.slopes ? a.slopes + h0 : nullptr, sm.add_one = a.add_one;
			const bool head_gate = a.gate && a.ges == 0; // one gate per head scales the probabilities; a gate per channel goes into the value product's epilogue
			sm.sink = a.sink ? a.sink + h0 : nullptr, sm.gate = head_gate ? a.gate + (size_t)(first + t0) * a.ldg + h0 : nullptr, sm.ldg = a.ldg;
			GemmExtra gx;
			if (a.gate && !head_gate) gx.gate = a.gate + (size_t)(first + t0) * a.ldg + (size_t)h0 * a.ghs, gx.ldgate = a.ldg, gx.gbs = a.ghs;
			run_kernel(s, kind, (double)a.group * Tb * Cp * (4 + 2 * px), 0, [&] { launch_k(s, k_seq_attn_softmax, dim3(Tb, a.group), 256, 0, sm); });
			gemm(s, s.att_p, (long)Cp * px, (long)Tb * Cp * px, s.att_vt, (long)Cp * px, 0, out + ((size_t)(first + t0) * a.heads + h0) * a.vd, (long)a.heads * a.vd, a.vd, Tb, a.vd,
			     a.split ? Cp + C : C, a.group, EPI_ACT, nullptr, kind, false, &gx);
		}
		t0 += Tb;
	}
}

void attention(Seq& s, int kind, AttArgs a, void* out, const SeqBatch& sb, double kv_rows, int longest) {
	a.skip = nullptr;
	bool rest = true;
	if (!s.m.exact && s.attn_products && s.n_on_products > 0) {
		const size_t n = (size_t)sb.N * a.heads * a.kd;
		if (a.split) run_kernel(s, KD_ELEMENT, n * 10.0, 0, [&] { launch_k(s, k_seq_split_q, cdiv(n, 256), 256, 0, (bf16*)s.a3, a.q, a.kd, (size_t)sb.N * a.heads); });
		else run_kernel(s, KD_ELEMENT, n * 6.0, 0, [&] { launch_k(s, k_seq_cast_cols<bf16>, cdiv(n, 256), 256, 0, (bf16*)s.a3, a.q, a.heads * a.kd, 0, a.heads * a.kd, sb.N); });
		for (int b = 0; b < sb.B; ++b)
			if (s.hb_count[b] >= kAttnGemmMin) attention_products(s, kind, a, (bf16*)out, sb, s.hb_slot[b], s.hb_start[b], s.hb_count[b], s.hb_pos0[b]);
		a.skip = s.d_skip;
		rest = s.n_on_products < sb.B;
	}
	if (!rest) return;
	const size_t smem = attn_smem(a.tile, a.kd);
	// few tokens over a long context: the keys of one (token, head tile) are shared out over several CTAs
	const int live = a.skip ? std::max(1, sb.N - s.tok_on_products) : sb.N; // tokens the fused kernel really serves (the others' CTAs leave at once)
	int span = a.window > 0 ? a.window + a.keep_first : 0;
	if (a.chunk > 0) span = span > 0 ? std::min(span, a.chunk) : a.chunk;
	a.nsplit = attn_nsplit(s, live, a.heads / a.tile, span, longest);
	ensure_part(s, (size_t)sb.N * a.heads * a.nsplit * (a.vd + 2));
	a.part = s.part;
	const dim3 grid(sb.N, a.heads / a.tile, a.nsplit);
	const double bytes = kv_rows * (a.heads / a.group) * (a.kc == a.vc ? a.kd : a.kd + a.vd) * 4.0;
	const double flops = 2.0 * kv_rows * a.heads * (a.kd + a.vd);
	run_kernel(s, kind, a.skip ? 0 : bytes, a.skip ? 0 : flops, [&] {
		if (s.m.exact) launch_k(s, k_seq_attention<float>, grid, ATT_THREADS, smem, a, (float*)out, sb);
		else launch_k(s, k_seq_attention<bf16>, grid, ATT_THREADS, smem, a, (bf16*)out, sb);
	});
	if (a.nsplit > 1)
		run_kernel(s, kind, 0, 0, [&] {
			if (s.m.exact) launch_k(s, k_seq_attention_merge<float>, dim3(sb.N, a.heads), 128, 0, a, (float*)out);
			else launch_k(s, k_seq_attention_merge<bf16>, dim3(sb.N, a.heads), 128, 0, a, (bf16*)out);
		});
}

void conv(Seq& s, const SeqLayer& L, RunState& r, ConvArgs& ca, const SeqBatch& sb) {
	const int units = ca.seg[0].heads + ca.seg[1].heads + ca.seg[2].heads;
	ca.proj = s.proj, ca.ldp = proj_stride(L), ca.w = (const bf16*)L.conv, ca.taps = L.taps, ca.channels = conv_channels(L), ca.state = r.conv, ca.eps = s.m.eps;
	ca.bias = (const bf16*)L.conv_b, ca.pcol = L.type == SEQ_MAMBA2 ? L.heads * L.vdim : 0; // Mamba-2: the channels start behind z
	const double bytes = (double)sb.N * ca.channels * 8;
	run_kernel(s, KD_CONV, bytes, 0, [&] { launch_k(s, k_seq_conv_heads, dim3(sb.N, cdiv(units, 4)), 128, 0, ca, sb); });
	if (L.taps > 1)
		run_kernel(s, KD_CONV, 0, 0, [&] { launch_k(s, k_seq_conv_state, dim3(cdiv(ca.channels, 128), sb.B), 128, 0, r.conv, s.proj, ca.ldp, L.taps, ca.channels, sb, ca.pcol); });
}

// how a sublayer's last product lands in the stream: serial blocks apply the Dynamic Tanh norm after the sublayer and add
// (EPI_DYT_RES into x); parallel blocks park the mixer's output (EPI_F32 into `mo`) and add it together with the feed-forward's
// (EPI_RES into x with res = mo), or add it alone when the layer has no feed-forward
struct OutEpi {
	int epi;
	const SeqNorm* nrm;
	float* dst;
	const float* res;
	float scale = 0.f; // != 0: factor on the product
	const SeqHyper* hc = nullptr; // hyper blocks: the routed feed-forward writes the streams itself (its weighted sum is formed in that kernel)
	const void* next_in = nullptr;      // ... and in the same kernel reads them for the sublayer that follows: its `in` weights and its norm
	const SeqNorm* next_norm = nullptr;
	const SeqNorm* post = nullptr;      // post-norm blocks: the norm the routed feed-forward's sum goes through on its way into the stream
};
// post-norm blocks: x += norm(y), y = base + the routed experts' sum; the new rows also leave in the activation type (hA), the next sublayer's input
template <typename AT>
void post_norm(Seq& s, const float* base, const HcMoe& moe, const SeqNorm& nm, int N) {
	const int W = s.m.width;
	run_kernel(s, KD_NORM, (double)N * W * (8.0 + (base ? 4 : 0) + (moe.y ? 4.0 * moe.top : 0) + act_size(s)), 0, [&] {
		if (W % 4 == 0) // a group of four neighbouring columns per thread up to 1024 columns, whole warps
			launch_k(s, k_seq_post_norm<AT, 4>, N, std::min(256, cdiv(W / 4, 32) * 32), 0, s.x, (AT*)s.hA, base, moe, (const bf16*)nm.w, s.m.norm_offset, s.m.eps, N, W);
		else launch_k(s, k_seq_post_norm<AT, 1>, N, std::min(256, cdiv(W, 32) * 32), 0, s.x, (AT*)s.hA, base, moe, (const bf16*)nm.w, s.m.norm_offset, s.m.eps, N, W);
	});
}
// write the streams from a sublayer's output; with next_in / next_norm also the normed input of the sublayer that follows (into hA)
template <typename AT>
void hc_write(Seq& s, const SeqHyper& hc, const float* base, const HcMoe& moe, int N, const void* next_in, const SeqNorm* next_norm) {
	const int W = s.m.width, S = s.streams;
	HcRead rd{next_norm ? s.hA : nullptr, (const bf16*)next_in, next_norm ? (const bf16*)next_norm->w : nullptr, s.m.norm_scalar ? 1 : W, s.m.norm_offset, s.m.eps};
	run_kernel(s, KD_HYPER, (double)N * W * (8.0 * S + 4 + (moe.y ? 4.0 * moe.top : 0) + (rd.out ? act_size(s) : 0)), 0, [&] {
		auto go = [&](auto kernel, int threads) { launch_k(s, kernel, N, threads, 0, s.x, base, (const bf16*)hc.mix, (const bf16*)hc.out, N, W, S, moe, (const AT*)s.hA, rd); };
		const int t4 = std::min(512, cdiv(W / 4, 32) * 32), t1 = std::min(1024, cdiv(W, 32) * 32);
		if (W % 4 == 0) { // four neighbouring columns per thread, one group per thread up to 2048 columns
			if (S <= 4) go(k_seq_hc_write<AT, 4, 4>, t4);
			else go(k_seq_hc_write<AT, 4, HC_MAX>, t4);
		} else if (S <= 4) go(k_seq_hc_write<AT, 1, 4>, t1);
		else go(k_seq_hc_write<AT, 1, HC_MAX>, t1);
	});
}
template <typename AT>
void out_product(Seq& s, const AT* X, const void* Wt, int N, int K, const OutEpi& oe, const void* bias = nullptr) {
	GemmExtra gx;
	gx.res = oe.res, gx.out_scale = oe.scale, gx.bias = bias; // the factor applies to product + bias
	gemm(s, X, K, 0, Wt, K, 0, oe.dst, s.m.width, 0, N, s.m.width, K, 1, oe.epi, oe.nrm, -1, true, &gx);
}

// the gated-linear-attention scan over a step's tokens: S <- diag(decay) S + k v^T, o = S^T q * qscale per (sequence, head); g names
// the inputs (columns of a matrix with row stride ld), the state and the output
void gla_launch(Seq& s, GlaArgs& g, const SeqBatch& sb, int ld) {
	const int N = sb.N, H = g.heads, D = g.dim, Dv = g.vdim;
	g.ldp = ld;
	g.vec = D % 4 == 0 && Dv % 4 == 0 && ld % 4 == 0 && g.qcol % 4 == 0 && g.kcol % 4 == 0 && g.vcol % 4 == 0 && ((uintptr_t)g.proj & 15) == 0; // 16-byte copies
	g.ldstate = gla_ldstate(D);
	// lanes per value column: more of them while sequences x heads x columns alone would leave SMs without a CTA
	int lanes = 4;
	while (lanes < 16 && (long)sb.B * H * cdiv(Dv * lanes, 128) < s.sms) lanes *= 2;
	const int R = gla_rows(D, lanes);
	const dim3 grid(sb.B, H, cdiv(Dv * lanes, 128));
	const size_t smem = gla_smem(R, lanes);
	run_kernel(s, KD_GLA, (double)N * H * (3.0 * D + 2.0 * Dv) * 4 + 2.0 * sb.B * H * D * Dv * 4, (double)N * H * D * Dv * 4.0, [&] {
		bool done = false;
		gla_each([&](auto r, auto p) {
			if (decltype(r)::value == R && decltype(p)::value == lanes) launch_k(s, k_seq_gla_scan<decltype(r)::value, decltype(p)::value>, grid, 128, smem, g, sb), done = true;
		});
		if (!done) CALM_FATAL("seq: no gated-linear-attention scan for %d key channels on %d lanes", D, lanes);
	});
}

template <typename AT>
void mixer_typed(Seq& s, const SeqLayer& L, RunState& r, const SeqBatch& sb, double kv_rows, int longest, const OutEpi& oe, const float* proj_in = nullptr, int ld_in = 0) {
	// proj_in: the mixer's input projection has been computed already (a pair's stacked product): its fp32 columns start there, row stride ld_in,
	// and a gated-linear-attention's decay input (its last rows) waits in a1 in the activation type
	const int N = sb.N, W = s.m.width, P = proj_in ? ld_in : proj_stride(L);
	const float* const proj = proj_in ? proj_in : s.proj;
	AT *hA = (AT*)s.hA, *a1 = (AT*)s.a1, *a2 = (AT*)s.a2;
	bool a1_ready = proj_in != nullptr;
	if (L.type != SEQ_PAIR && !proj_in) {
		// one product for everything that reads the normed input: the mixer's rows, and in parallel blocks the router's rows (fp32, behind
		// the mixer's) or the dense unit's up rows (leaving as relu^2 in the activation type)
		GemmExtra gx;
		gx.bias = L.b_in;
		int M = (int)in_rows(L);
		if (L.in_tail > 0 && L.ff_kind == SEQ_FF_MOE) M += L.in_tail;
		if (L.in_tail > 0 && L.ff_kind == SEQ_FF_RELU2) gx.split = M, gx.Y2 = s.ah, gx.ldy2 = L.ff, M += L.in_tail;
		if (L.in_tail == 0 && L.type == SEQ_GLA) // the decay's low-rank input (the last rows) leaves the epilogue in the activation type, ready for its second product
			gx.split = M - L.a_rank, gx.split_act = 1, gx.Y2 = a1, gx.ldy2 = L.a_rank, a1_ready = true;
		gemm(s, hA, W, 0, L.w_in, W, 0, s.proj, P, 0, N, M, W, 1, EPI_F32, nullptr, -1, true, &gx);
	}
	if (L.type == SEQ_LATENT) {
		const int H = L.heads, D = L.dim, Dv = L.vdim, Rq = L.q_rank, Rk = L.kv_rank;
		RmsSeg sq{0, Rq, (const bf16*)L.dq_norm}, sc{Rq, Rk, (const bf16*)L.dkv_norm};
		run_kernel(s, KD_NORM, (double)N * (Rq + Rk) * 8, 0,
		           [&] { launch_k(s, k_seq_latent_norm<AT>, dim3(cdiv(N, 4), 2), 128, 0, s.proj, P, sq, sc, a1, r.cache_a, sb, s.m.eps); });
		gemm(s, a1, Rq, 0, L.w_uq, Rq, 0, a2, (long)H * D, 0, N, H * D, Rq, 1, EPI_ACT);
		// the key up-projection moves to the query side: q'_h = W_uk,h^T q_h, so scores and values are taken on the cached latent itself
		gemm(s, a2, (long)H * D, D, L.w_ukT, D, (long)Rk * D, s.f[0], (long)H * Rk, Rk, N, Rk, D, H, EPI_F32);
		AttArgs a;
		a.q = s.f[0], a.kc = a.vc = r.cache_a, a.kld = a.vld = Rk, a.heads = H, a.group = H, a.tile = attn_tile(H, Rk, Rk), a.kd = a.vd = Rk, a.window = 0;
		a.scale = L.scale, a.sink = nullptr, a.gate = s.proj + Rq + Rk, a.ldg = P, a.ghs = 1, a.ges = 0, a.keep_first = 0;
		attention(s, KD_ATTN_LATENT, a, a1, sb, kv_rows, longest);
		gemm(s, a1, (long)H * Rk, Rk, L.w_uv, Rk, (long)Dv * Rk, a2, (long)H * Dv, Dv, N, Dv, Rk, H, EPI_ACT);
		out_product<AT>(s, a2, L.w_o, N, H * Dv, oe, L.b_o);
	} else if (L.type == SEQ_DELTA) {
		const int H = L.heads, G = L.kv_heads, D = L.dim, Dv = L.vdim;
		const int cq = 0, ck = G * D, cv = 2 * G * D, cb = cv + H * Dv, ca1 = cb + H, cg1 = ca1 + L.a_rank;
		ConvArgs ca;
		ca.seg[0] = ConvSeg{cq, G, D, 1, 1, 1.f / sqrtf((float)D), 0, s.f[0]};
		ca.seg[1] = ConvSeg{ck, G, D, 1, 1, 1.f, 0, s.f[1]};
		ca.seg[2] = ConvSeg{cv, H, Dv, 1, 0, 1.f, 0, s.f[2]};
		conv(s, L, r, ca, sb);
		const int lr = L.a_rank + L.g_rank;
		run_kernel(s, KD_ELEMENT, (double)N * lr * 6, 0, [&] { launch_k(s, k_seq_cast_cols<AT>, cdiv((long)N * lr, 256), 256, 0, a1, s.proj, P, ca1, lr, N); });
		gemm(s, a1, lr, 0, L.w_a2, L.a_rank, 0, s.f[3], (long)H * D, 0, N, H * D, L.a_rank, 1, EPI_F32);
		gemm(s, a1 + L.a_rank, lr, 0, L.w_g2, L.g_rank, 0, s.f[4], (long)H * Dv, 0, N, H * Dv, L.g_rank, 1, EPI_F32);
		(void)cg1;
		DeltaArgs d;
		d.q = s.f[0], d.k = s.f[1], d.v = s.f[2], d.proj = s.proj, d.ldp = P, d.bcol = cb, d.dt = s.f[3], d.a_log = (const bf16*)L.a_log, d.dt_bias = (const bf16*)L.dt_bias;
		d.state = r.delta, d.o = s.f[5], d.heads = H, d.kv_heads = G, d.dim = D, d.vdim = Dv;
		const size_t smem = ((size_t)D * Dv + 3 * D) * sizeof(float);
		const int threads = std::max(64, cdiv(Dv, 32) * 32);
		const size_t smem_reg = 2 * (size_t)DELTA_TB * (3 * (D + 16) + ((Dv + 4) & ~3)) * sizeof(float);
		const int threads_reg = std::max(256, cdiv(4 * Dv, 32) * 32); // two staging rounds cover DELTA_TB * ((3 D + Dv) / 4 + 1) items
		const bool reg = (D == 32 || D == 64 || D == 128) && 4 * Dv <= 512 && Dv % 4 == 0 && !getenv("CALM_B200_SEQ_DELTA_SMEM");
		run_kernel(s, KD_DELTA, (double)N * H * (3.0 * D + 2.0 * Dv) * 4 + 2.0 * sb.B * H * D * Dv * 4, (double)N * H * D * Dv * 6.0, [&] {
			const dim3 grid(sb.B, H);
			if (reg && D == 32) launch_k(s, k_seq_delta_scan_reg<32>, grid, threads_reg, smem_reg, d, sb);
			else if (reg && D == 64) launch_k(s, k_seq_delta_scan_reg<64>, grid, threads_reg, smem_reg, d, sb);
			else if (reg && D == 128) launch_k(s, k_seq_delta_scan_reg<128>, grid, threads_reg, smem_reg, d, sb);
			else launch_k(s, k_seq_delta_scan, dim3(sb.B, H), threads, smem, d, sb);
		});
		run_kernel(s, KD_NORM, (double)N * H * Dv * 10, 0,
		           [&] { launch_k(s, k_seq_delta_out<AT>, cdiv((long)N * H, 4), 128, 0, a2, s.f[5], s.f[4], H * Dv, (const bf16*)L.out_norm, N, H, Dv, s.m.eps, 0); });
		out_product<AT>(s, a2, L.w_o, N, H * Dv, oe, L.b_o);
	} else if (L.type == SEQ_GQA) {
		const int H = L.heads, G = L.kv_heads, D = L.dim, Dv = L.vdim;
		QkArgs qa;
		qa.proj = proj, qa.ldp = P, qa.heads = H, qa.kv_heads = G, qa.dim = D, qa.vdim = Dv, qa.qw = (const bf16*)L.q_norm, qa.kw = (const bf16*)L.k_norm, qa.eps = s.m.eps;
		const auto rt = s.rot.find(&L);
		qa.rot_dims = rt == s.rot.end() ? 0 : L.rot_dims, qa.freq = rt == s.rot.end() ? nullptr : rt->second.first, qa.mag = rt == s.rot.end() ? 1.f : rt->second.second, qa.q = s.f[0], qa.kc = r.cache_a, qa.vc = r.cache_b;
		qa.v_norm = L.v_norm, qa.per_head = L.qk_per_head;
		const size_t qk_smem = ((size_t)2 * std::max(L.rot_dims / 2, 1) + H + G) * sizeof(float);
		run_kernel(s, KD_QK, (double)N * (H * D + G * D + G * Dv) * 8, 0, [&] { launch_k(s, k_seq_qk_rope, N, 256, qk_smem, qa, sb); });
		AttArgs a;
		a.q = s.f[0], a.kc = r.cache_a, a.vc = r.cache_b, a.kld = G * D, a.vld = G * Dv, a.heads = H, a.group = H / G, a.tile = attn_tile(H / G, D, Dv), a.kd = D, a.vd = Dv;
		a.window = L.window, a.keep_first = L.window > 0 ? L.keep_first : 0, a.scale = L.scale, a.sink = nullptr;
		a.gate = L.no_gate ? nullptr : proj + H * D + G * D + G * Dv, a.ldg = P, a.ghs = L.gate_per_head ? 1 : Dv, a.ges = L.gate_per_head ? 0 : 1; // a sigmoid gate per output channel (or per head), from the same stacked projection
		a.chunk = L.chunk, a.slopes = L.dist_bias ? r.slopes : nullptr, a.add_one = L.add_one;
		const int span = attn_span(L);
		a.split = L.scores_f32;
		attention(s, KD_ATTN_WINDOW, a, a2, sb, span > 0 ? std::min(kv_rows, (double)N * span) : kv_rows, longest);
		out_product<AT>(s, a2, L.w_o, N, H * Dv, oe, L.b_o);
	} else if (L.type == SEQ_PAIR) {
		// two mixers on the same normed input: the first one's product lands scaled in the destination, the second one's is added scaled
		if (oe.epi != EPI_F32) CALM_FATAL("seq: a pair writes its sum to a buffer of its own");
		OutEpi first = oe, second = oe;
		first.scale = L.pair_scale[0], second.epi = EPI_RES, second.res = nullptr, second.scale = L.pair_scale[1];
		if (L.w_in) {
			// both mixers' input rows are one matrix (the first's rows padded to a multiple of 8, then the second's): one product; a
			// gated-linear-attention in second place sends its decay input (the last rows) out in the activation type
			const int off = pair_offset(L), M = off + (int)in_rows(L.pair[1]), ld = pair_stride(L);
			GemmExtra gx;
			gx.bias = L.b_in;
			if (L.pair[1].type == SEQ_GLA) gx.split = M - L.pair[1].a_rank, gx.split_act = 1, gx.Y2 = a1, gx.ldy2 = L.pair[1].a_rank;
			gemm(s, hA, W, 0, L.w_in, W, 0, s.proj, ld, 0, N, M, W, 1, EPI_F32, nullptr, -1, true, &gx);
			mixer_typed<AT>(s, L.pair[0], r.sub[0], sb, kv_rows, longest, first, s.proj, ld);
			mixer_typed<AT>(s, L.pair[1], r.sub[1], sb, kv_rows, longest, second, s.proj + off, ld);
			return;
		}
		mixer_typed<AT>(s, L.pair[0], r.sub[0], sb, kv_rows, longest, first);
		mixer_typed<AT>(s, L.pair[1], r.sub[1], sb, kv_rows, longest, second);
	} else if (is_lin(L)) {
		// mLSTM, HGRN2, Mamba-2: gates and inputs are prepared in fp32, the recurrence is the gated-linear-attention scan, a read-out kernel finishes
		const int H = L.heads, D = L.dim, Dv = L.vdim, Vs = lin_vs(L), ldl = 2 * H * D + H * Vs;
		LinPack lp;
		memset(&lp, 0, sizeof(lp));
		lp.proj = s.proj, lp.ldp = P, lp.lin = s.lin, lp.decay = s.f[3], lp.heads = H, lp.dim = D, lp.vdim = Dv, lp.vs = Vs;
		LinOut lo;
		memset(&lo, 0, sizeof(lo));
		lo.o = s.f[5], lo.ldo = H * Vs, lo.ohs = Vs, lo.heads = H, lo.vdim = Dv, lo.unit = Dv, lo.w = (const bf16*)L.out_norm, lo.eps = s.m.eps, lo.mul = 1.f;
		float qscale = 1.f;
		if (L.type == SEQ_MLSTM) {
			const int cq = 0, ck = H * D, cv = 2 * H * D, cg = cv + H * Dv, ci = cg + H * Dv, cf = ci + H;
			MlstmGates mg{s.proj, P, ci, cf, H, L.gate_cap, r.mstate, s.f[0], s.f[1], s.f[2]};
			run_kernel(s, KD_LINPREP, (double)N * H * 20, 0, [&] { launch_k(s, k_seq_mlstm_gates, dim3(sb.B, H), 32, 0, mg, sb); });
			lp.mode = LIN_MLSTM, lp.qcol = cq, lp.kcol = ck, lp.vcol = cv, lp.keep = s.f[0], lp.take = s.f[1];
			lo.w_mod = H * Dv, lo.gate = s.proj + cg, lo.ldg = P, lo.gate_mode = 1, lo.m_t = s.f[2];
			qscale = 1.f / sqrtf((float)D);
		} else if (L.type == SEQ_HGRN2) {
			lp.mode = LIN_HGRN2, lp.qcol = 0, lp.kcol = H * D, lp.vcol = 2 * H * D, lp.lower = (const bf16*)L.lower;
			lo.w_mod = Dv;
		} else {
			const int G = L.kv_heads, inner = H * Dv;
			ConvArgs ca;
			ca.seg[0] = ConvSeg{0, H, Dv, 1, 0, 1.f, 0, s.f[0]};
			ca.seg[1] = ConvSeg{inner, G, D, 1, 0, 1.f, 0, s.f[1]};
			ca.seg[2] = ConvSeg{inner + G * D, G, D, 1, 0, 1.f, 0, s.f[2]};
			conv(s, L, r, ca, sb);
			lp.mode = LIN_MAMBA2, lp.xs = s.f[0], lp.bs = s.f[1], lp.cs = s.f[2], lp.dtcol = 2 * inner + 2 * G * D, lp.groups = G;
			lp.dt_bias = (const bf16*)L.dt_bias, lp.a_log = (const bf16*)L.a_log;
			lo.unit = inner / L.norm_groups, lo.w_mod = inner, lo.gate = s.proj, lo.ldg = P, lo.gate_mode = 3, lo.skip = s.f[0], lo.skip_w = (const bf16*)L.skip_d;
		}
		run_kernel(s, KD_LINPREP, (double)N * (ldl + H * D) * 8, 0, [&] { launch_k(s, k_seq_lin_pack, dim3(N, H), 64, 0, lp, N); });
		GlaArgs g;
		g.proj = s.lin, g.qcol = 0, g.kcol = H * D, g.vcol = 2 * H * D, g.decay = s.f[3], g.qscale = qscale;
		g.state = r.delta, g.o = s.f[5], g.heads = H, g.dim = D, g.vdim = Vs;
		gla_launch(s, g, sb, ldl);
		const long units = (long)N * (H * Dv / lo.unit);
		run_kernel(s, KD_NORM, (double)N * H * Dv * 10, 0, [&] { launch_k(s, k_seq_lin_out<AT>, cdiv(units, 4), 128, 0, a2, lo, N); });
		out_product<AT>(s, a2, L.w_o, N, H * Dv, oe, L.b_o);
	} else if (L.type == SEQ_GLA) {
		const int H = L.heads, D = L.dim, Dv = L.vdim;
		const int cq = 0, ck = H * D, cv = 2 * H * D, cg = cv + H * Dv, ca1 = cg + H * Dv;
		if (!a1_ready)
			run_kernel(s, KD_ELEMENT, (double)N * L.a_rank * 6, 0, [&] { launch_k(s, k_seq_cast_cols<AT>, cdiv((long)N * L.a_rank, 256), 256, 0, a1, proj, P, ca1, L.a_rank, N); });
		{
			GemmExtra gx; // the decay sigmoid(.)^(1/tau) leaves the product's epilogue in fp32
			gx.bias = L.b_a2, gx.epi_f = 1.f / L.tau;
			gemm(s, a1, L.a_rank, 0, L.w_a2, L.a_rank, 0, s.f[3], (long)H * D, 0, N, H * D, L.a_rank, 1, EPI_DECAY, nullptr, -1, true, &gx);
		}
		GlaArgs g;
		g.proj = proj, g.ldp = P, g.qcol = cq, g.kcol = ck, g.vcol = cv, g.decay = s.f[3], g.qscale = 1.f / sqrtf((float)D);
		g.state = r.delta, g.o = s.f[5], g.heads = H, g.dim = D, g.vdim = Dv;
		gla_launch(s, g, sb, P);
		run_kernel(s, KD_NORM, (double)N * H * Dv * 10, 0, [&] {
			launch_k(s, k_seq_delta_out<AT>, cdiv((long)N * H, 4), 128, 0, a2, s.f[5], proj + cg, P, (const bf16*)L.out_norm, N, H, Dv, s.m.eps, 1);
		});
		out_product<AT>(s, a2, L.w_o, N, H * Dv, oe, L.b_o);
	} else {
		const int H = L.heads, G = L.kv_heads, D = L.dim, Dv = L.vdim;
		ConvArgs ca;
		ca.seg[0] = ConvSeg{0, H, D, 0, 2, 1.f, 0, s.f[0]};
		ca.seg[1] = ConvSeg{H * D, G, D, 0, 2, 1.f, 1, r.cache_a};
		ca.seg[2] = ConvSeg{H * D + G * D, G, Dv, 0, 0, 1.f, 1, r.cache_b};
		conv(s, L, r, ca, sb);
		AttArgs a;
		a.q = s.f[0], a.kc = r.cache_a, a.vc = r.cache_b, a.kld = G * D, a.vld = G * Dv, a.heads = H, a.group = H / G, a.tile = attn_tile(H / G, D, Dv), a.kd = D, a.vd = Dv;
		a.window = L.window, a.scale = L.scale, a.sink = (const bf16*)L.sink, a.gate = nullptr, a.ldg = 0, a.ghs = 1, a.ges = 0, a.keep_first = 0;
		attention(s, KD_ATTN_WINDOW, a, a2, sb, L.window > 0 ? std::min(kv_rows, (double)N * L.window) : kv_rows, longest);
		out_product<AT>(s, a2, L.w_o, N, H * Dv, oe, L.b_o);
	}
}

// the feed-forward of a layer on the normed rows in hA
template <typename AT>
void feed_forward(Seq& s, const SeqLayer& L, const SeqBatch& sb, const OutEpi& oe) {
	const int N = sb.N, W = s.m.width;
	AT *hA = (AT*)s.hA, *a2 = (AT*)s.a2;
	if (L.ff_kind == SEQ_FF_CLAMPED) {
		gemm(s, hA, W, 0, L.w_gate_up, W, 0, s.proj, 2L * L.ff, 0, N, 2 * L.ff, W, 1, EPI_F32);
		run_kernel(s, KD_ELEMENT, (double)N * L.ff * (8 + sizeof(AT)), 0,
		           [&] { launch_k(s, k_seq_ff_act<AT>, cdiv((long)N * L.ff, 256), 256, 0, a2, s.proj, L.ff, N, L.limit, 0, 2 * L.ff); });
		out_product<AT>(s, a2, L.w_down, N, L.ff, oe);
	} else if (L.ff_kind == SEQ_FF_GATED) {
		gemm(s, hA, W, 0, L.w_gate_up, W, 0, s.proj, 2L * L.ff, 0, N, 2 * L.ff, W, 1, EPI_F32);
		run_kernel(s, KD_ELEMENT, (double)N * L.ff * (8 + sizeof(AT)), 0,
		           [&] { launch_k(s, k_seq_ff_act<AT>, cdiv((long)N * L.ff, 256), 256, 0, a2, s.proj, L.ff, N, 0.f, L.ff_act == SEQ_ACT_GELU_TANH ? 2 : 1, 2 * L.ff); });
		out_product<AT>(s, a2, L.w_down, N, L.ff, oe);
	} else if (L.ff_kind == SEQ_FF_RELU2) {
		if (L.in_tail > 0) { // the up rows rode in the mixer's input product
			out_product<AT>(s, (const AT*)s.ah, L.w_down, N, L.ff, oe);
			return;
		}
		gemm(s, hA, W, 0, L.w_gate_up, W, 0, a2, L.ff, 0, N, L.ff, W, 1, EPI_ACT_RELU2); // relu(up)^2 leaves the product's epilogue in the activation type
		out_product<AT>(s, a2, L.w_down, N, L.ff, oe);
	} else {
		// routed experts: logits -> choices and weights -> pairs grouped by expert -> two grouped products around the unit -> weighted sum
		const int E = L.experts, Et = E + L.ident, top = L.top, pairs = N * top, ff = L.ff;
		const float* logits = s.proj;
		int ldl = Et;
		const int sf = L.shared_ff, ldsh = 2 * sf + (L.w_router ? 0 : Et);
		const bool r2 = L.expert_act == 1;
		// relu^2 units: the shared unit's first product is [gate row | router rows | up rows]; the up rows leave its epilogue as relu(.)^2 in the
		// activation type, the gate's and the router's columns stay fp32
		const int shc = (L.shared_gate ? 1 : 0) + (L.w_router ? 0 : Et);
		if (r2 && sf > 0) {
			GemmExtra sx;
			if (shc > 0) {
				sx.split = shc, sx.Y2 = a2, sx.ldy2 = sf;
				gemm(s, hA, W, 0, L.w_sh_gate_up, W, 0, s.fsh, shc, 0, N, shc + sf, W, 1, EPI_F32, nullptr, -1, true, &sx);
			} else gemm(s, hA, W, 0, L.w_sh_gate_up, W, 0, a2, sf, 0, N, sf, W, 1, EPI_ACT_RELU2);
		}
		if (r2 && sf > 0 && !L.w_router) logits = s.fsh + (L.shared_gate ? 1 : 0), ldl = shc;
		else if (L.in_tail > 0) logits = s.proj + in_rows(L), ldl = proj_stride(L); // the router's rows rode in the mixer's input product
		else if (!L.w_router) { // the router's rows ride behind the shared unit's [gate | up]: one product for everything that reads the normed input
			gemm(s, hA, W, 0, L.w_sh_gate_up, W, 0, s.fsh, ldsh, 0, N, ldsh, W, 1, EPI_F32);
			logits = s.fsh + 2 * sf, ldl = ldsh;
		} else {
			GemmExtra rx;
			rx.bias = L.b_router;
			gemm(s, hA, W, 0, L.w_router, W, 0, s.proj, Et, 0, N, Et, W, 1, EPI_F32, nullptr, -1, true, &rx);
		}
		const float rscale = L.route_scale != 0.f ? L.route_scale : 1.f;
		// identity experts get groups of their own behind the real ones: their rows are placed but no product runs over them
		if (N <= MOE_SMALL_TOKENS) { // a decode step: choices and groups in one launch
			run_kernel(s, KD_ROUTE, (double)N * Et * 4 + (double)pairs * 4 * Et, 0, [&] {
				launch_k(s, k_seq_moe_route_group, 1, 256, 0, logits, ldl, Et, top, N, s.moe_sel, s.moe_wt, L.route_mode, (const bf16*)L.correction, rscale, s.moe_seg, s.moe_perm, s.moe_inv);
			});
		} else {
			run_kernel(s, KD_ROUTE, (double)N * Et * 4, 0,
			           [&] { launch_k(s, k_seq_moe_route, cdiv(N, 4), 128, 0, logits, ldl, Et, top, N, s.moe_sel, s.moe_wt, L.route_mode, (const bf16*)L.correction, rscale); });
			run_kernel(s, KD_ROUTE, (double)pairs * 4 * Et, 0, [&] { launch_k(s, k_seq_moe_group, Et, 256, 0, s.moe_sel, pairs, Et, s.moe_seg, s.moe_perm, s.moe_inv); });
		}
		run_kernel(s, KD_ELEMENT, (double)pairs * W * 2 * sizeof(AT), 0,
		           [&] { launch_k(s, k_seq_moe_gather<AT>, cdiv((long)pairs * W, 256), 256, 0, (AT*)s.moe_x, hA, s.moe_perm, top, pairs, W); });
		GemmExtra gx;
		gx.seg = s.moe_seg, gx.x_rows = pairs;
		if (r2) {
			// relu^2 experts: relu(w u)^2 leaves the grouped up product's epilogue (w = the pair's weight when it multiplies the expert's input: the
			// up projection is linear, so w h becomes w u in fp32), then the grouped down product; the shared unit's down product takes the
			// sigmoid of its gate column as a factor per row
			GemmExtra ux = gx;
			if (L.weight_input) ux.rs = s.moe_wt, ux.rs_idx = s.moe_perm;
			gemm(s, s.moe_x, W, 0, L.w_gate_up, W, (long)ff * W, s.moe_a, ff, 0, N, ff, W, E, EPI_ACT_RELU2, nullptr, -1, true, &ux);
			gemm(s, s.moe_a, ff, 0, L.w_down, ff, (long)W * ff, s.moe_d, W, 0, N, W, ff, E, EPI_F32, nullptr, -1, true, &gx);
			if (sf > 0) {
				GemmExtra dx;
				if (L.shared_gate) dx.rs = s.fsh, dx.rs_ld = shc, dx.rs_act = 1;
				gemm(s, a2, sf, 0, L.w_sh_down, sf, 0, s.mo, W, 0, N, W, sf, 1, EPI_F32, nullptr, -1, true, &dx);
			}
			post_norm<AT>(s, sf > 0 ? s.mo : nullptr, HcMoe{s.moe_d, s.moe_inv, s.moe_sel, L.weight_input ? nullptr : s.moe_wt, top, E}, *oe.post, N);
			return;
		}
		gemm(s, s.moe_x, W, 0, L.w_gate_up, W, 2L * ff * W, s.moe_y, 2L * ff, 0, N, 2 * ff, W, E, EPI_F32, nullptr, -1, true, &gx);
		if (oe.hc) {
			// hyper blocks: the shared unit's product is the base of y, the routed sum is formed while the streams are written; the two units'
			// activations are one launch
			if (sf > 0) {
				if (L.w_router) gemm(s, hA, W, 0, L.w_sh_gate_up, W, 0, s.fsh, ldsh, 0, N, ldsh, W, 1, EPI_F32);
				FfPair fp{{s.moe_y, s.fsh}, {s.moe_a, a2}, {ff, sf}, {pairs, N}, {2 * ff, ldsh}};
				run_kernel(s, KD_ELEMENT, ((double)pairs * ff + (double)N * sf) * (8 + sizeof(AT)), 0,
				           [&] { launch_k(s, k_seq_ff_act2<AT>, cdiv((long)pairs * ff + (long)N * sf, 256), 256, 0, fp); });
			} else
				run_kernel(s, KD_ELEMENT, (double)pairs * ff * (8 + sizeof(AT)), 0,
				           [&] { launch_k(s, k_seq_ff_act<AT>, cdiv((long)pairs * ff, 256), 256, 0, (AT*)s.moe_a, s.moe_y, ff, pairs, 0.f, 1, 2 * ff); });
			gemm(s, s.moe_a, ff, 0, L.w_down, ff, (long)W * ff, s.moe_d, W, 0, N, W, ff, E, EPI_F32, nullptr, -1, true, &gx);
			if (sf > 0) gemm(s, a2, sf, 0, L.w_sh_down, sf, 0, s.mo, W, 0, N, W, sf, 1, EPI_F32);
			hc_write<AT>(s, *oe.hc, sf > 0 ? s.mo : nullptr, HcMoe{s.moe_d, s.moe_inv, s.moe_sel, s.moe_wt, top, E}, N, oe.next_in, oe.next_norm);
			return;
		}
		run_kernel(s, KD_ELEMENT, (double)pairs * ff * (8 + sizeof(AT)), 0,
		           [&] { launch_k(s, k_seq_ff_act<AT>, cdiv((long)pairs * ff, 256), 256, 0, (AT*)s.moe_a, s.moe_y, ff, pairs, 0.f, 1, 2 * ff); });
		gemm(s, s.moe_a, ff, 0, L.w_down, ff, (long)W * ff, s.moe_d, W, 0, N, W, ff, E, EPI_F32, nullptr, -1, true, &gx);
		if (oe.post) { // post-norm blocks: the weighted sum is formed by the kernel that norms it and adds it to the stream
			post_norm<AT>(s, nullptr, HcMoe{s.moe_d, s.moe_inv, s.moe_sel, s.moe_wt, top, E}, *oe.post, N);
			return;
		}
		run_kernel(s, KD_ELEMENT, (double)N * W * (8 + 4.0 * top) + (oe.res ? (double)N * W * 4 : 0), 0, [&] {
			launch_k(s, k_seq_moe_combine<AT>, cdiv((long)N * W, 256), 256, 0, oe.dst, oe.res, s.moe_d, s.moe_inv, s.moe_wt, top, N, W, s.moe_sel, E, (const AT*)hA, 0);
		});
	}
}

// one run of a layer: norm, mixer, feed-forward, in the model's block form
template <typename AT>
void layer_typed(Seq& s, const SeqLayer& L, RunState& r, const SeqBatch& sb, double kv_rows, int longest, const SeqLayer* next) {
	const int N = sb.N;
	if (s.m.block == SEQ_BLOCK_HYPER) {
		// per sublayer: read the streams (u = sum in[s] x_s, normed), run it into `mo`, write all streams from the old ones and the result.
		// Only the first read of a step is a kernel of its own: every write also does the read of the sublayer that follows it.
		const HcMoe none{nullptr, nullptr, nullptr, nullptr, 0, 0};
		if (!s.h_ready) hc_read(s, s.hA, nullptr, L.hc1.in, L.norm1, N);
		const void* after_in = next ? next->hc1.in : nullptr;
		const SeqNorm* after_norm = next ? &next->norm1 : nullptr;
		mixer_typed<AT>(s, L, r, sb, kv_rows, longest, OutEpi{EPI_F32, nullptr, s.mo, nullptr});
		if (L.ff > 0) {
			hc_write<AT>(s, L.hc1, s.mo, none, N, L.hc2.in, &L.norm2);
			OutEpi oe{EPI_F32, nullptr, s.mo, nullptr};
			if (L.ff_kind == SEQ_FF_MOE) oe.hc = &L.hc2, oe.next_in = after_in, oe.next_norm = after_norm;
			feed_forward<AT>(s, L, sb, oe);
			if (!oe.hc) hc_write<AT>(s, L.hc2, s.mo, none, N, after_in, after_norm);
		} else hc_write<AT>(s, L.hc1, s.mo, none, N, after_in, after_norm);
		s.h_ready = next != nullptr;
		return;
	}
	if (s.m.block == SEQ_BLOCK_POST) {
		// the sublayers read the stream itself: hA holds its rows in the activation type, written by the kernel that last changed them
		const HcMoe none{nullptr, nullptr, nullptr, nullptr, 0, 0};
		if (!s.h_ready) {
			const size_t n = (size_t)N * s.m.width;
			run_kernel(s, KD_ELEMENT, n * (4.0 + sizeof(AT)), 0, [&] { launch_k(s, k_seq_cast_cols<AT>, cdiv(n, 256), 256, 0, (AT*)s.hA, s.x, s.m.width, 0, s.m.width, N); });
			s.h_ready = true;
		}
		mixer_typed<AT>(s, L, r, sb, kv_rows, longest, OutEpi{EPI_F32, nullptr, s.mo, nullptr});
		post_norm<AT>(s, s.mo, none, L.norm1, N);
		if (L.ff > 0) {
			OutEpi oe{EPI_F32, nullptr, s.mo, nullptr};
			oe.post = &L.norm2;
			feed_forward<AT>(s, L, sb, oe);
			if (L.ff_kind != SEQ_FF_MOE) post_norm<AT>(s, s.mo, none, L.norm2, N);
		}
		return;
	}
	norm(s, s.hA, s.x, nullptr, L.norm1, N);
	if (s.m.block == SEQ_BLOCK_SERIAL) {
		mixer_typed<AT>(s, L, r, sb, kv_rows, longest, OutEpi{EPI_DYT_RES, &L.norm1b, s.x, nullptr});
		if (L.ff > 0) {
			norm(s, s.hA, s.x, nullptr, L.norm2, N);
			feed_forward<AT>(s, L, sb, OutEpi{EPI_DYT_RES, &L.norm2b, s.x, nullptr});
		}
	} else if (L.ff > 0) { // x += mixer(h) + ff(h): the mixer's output waits in `mo` for the feed-forward's last kernel
		mixer_typed<AT>(s, L, r, sb, kv_rows, longest, OutEpi{EPI_F32, nullptr, s.mo, nullptr});
		feed_forward<AT>(s, L, sb, OutEpi{EPI_RES, nullptr, s.x, s.mo});
	} else {
		mixer_typed<AT>(s, L, r, sb, kv_rows, longest, OutEpi{EPI_RES, nullptr, s.x, nullptr});
	}
}

// every launch of one step, in order
void forward(Seq& s, const SeqBatch& sb, int n_want, double kv_rows, int longest) {
	const SeqModel& m = s.m;
	const int N = sb.N;
	const bool looped = m.loop_times > 1;
	s.h_ready = false;
	run_kernel(s, KD_EMBED, (double)N * m.width * (2.0 + (m.pos_table ? 2.0 : 0.0) + (m.bigram ? 2.0 : 0.0) + 4.0 * s.streams + (looped ? 4.0 : 0.0)), 0,
	           [&] { launch_k(s, k_seq_embed, N, 128, 0, s.x, looped ? s.x0 : nullptr, (const bf16*)m.embed, s.d_tok, N, m.width, m.embed_scale != 0.f ? m.embed_scale : 1.f, (const bf16*)m.pos_table, s.d_tpos, s.streams,
	                          EmbedBigram{(const bf16*)m.bigram, s.d_tprev, m.bigram_buckets, m.bigram_mul_prev, m.bigram_mul_cur}); });
	for (size_t ri = 0; ri < s.runs.size(); ++ri) {
		RunState& r = s.runs[ri];
		const SeqLayer& L = s.layers[r.layer];
		if (r.readd) {
			const size_t n = (size_t)N * m.width;
			run_kernel(s, KD_ELEMENT, n * 12.0, 0, [&] { launch_k(s, k_seq_add, cdiv(n, 256), 256, 0, s.x, s.x0, n); });
		}
		const SeqLayer* next = ri + 1 < s.runs.size() && !s.runs[ri + 1].readd ? &s.layers[s.runs[ri + 1].layer] : nullptr;
		if (m.exact) layer_typed<float>(s, L, r, sb, kv_rows, longest, next);
		else layer_typed<bf16>(s, L, r, sb, kv_rows, longest, next);
		if (s.trace) { // the residual stream after this run (the sum of the streams when there are several)
			const size_t n = (size_t)N * m.width;
			launch_k(s, k_seq_stream_sum, cdiv(n, 256), 256, 0, s.trace_buf + ri * n, s.x, N, m.width, s.streams);
			CUDA_CHECK(cudaGetLastError());
		}
	}
	if (n_want) {
		if (m.block == SEQ_BLOCK_HYPER) hc_read(s, s.hW, s.d_want, nullptr, m.final_norm, n_want);
		else norm(s, s.hW, s.x, s.d_want, m.final_norm, n_want);
		GemmExtra lx;
		lx.out_scale = m.logit_scale != 1.f ? m.logit_scale : 0.f; // 0: no factor
		gemm(s, s.hW, m.width, 0, m.head, m.width, 0, s.logits, m.vocab, 0, n_want, m.vocab, m.width, 1, EPI_F32, nullptr, -1, true, &lx);
	}
}

// One decoded token per sequence: the launch list depends only on the batch size, the rows wanted and how many CTAs share the keys
// of each attention run, so it is captured once per such key and replayed (the batch description, page table and tokens are data).
void forward_decode_graph(Seq& s, const SeqBatch& sb, int n_want, double kv_rows, int longest) {
	std::vector<int> key = {sb.N, n_want};
	size_t part_need = 0;
	auto one = [&](const SeqLayer& L) {
		if (L.type != SEQ_LATENT && L.type != SEQ_WINDOW && L.type != SEQ_GQA) return; // recurrent mixers: nothing to share out
		const bool lat = L.type == SEQ_LATENT;
		const int group = lat ? L.heads : L.heads / L.kv_heads, kd = lat ? L.kv_rank : L.dim, vd = lat ? L.kv_rank : L.vdim;
		const int ns = attn_nsplit(s, sb.N, L.heads / attn_tile(group, kd, vd), attn_span(L), longest);
		key.push_back(ns);
		part_need = std::max(part_need, (size_t)sb.N * L.heads * ns * (vd + 2));
	};
	for (const RunState& r : s.runs) {
		const SeqLayer& L = s.layers[r.layer];
		if (L.type == SEQ_PAIR) one(L.pair[0]), one(L.pair[1]);
		else one(L);
	}
	ensure_part(s, part_need); // no allocation inside a capture
	auto it = s.graphs.find(key);
	if (it == s.graphs.end()) {
		if (s.graphs.size() > 256) drop_graphs(s);
		const uint64_t before = g_seq_launches;
		cudaGraph_t graph = nullptr;
		cudaGraphExec_t exec = nullptr;
		CUDA_CHECK(cudaStreamBeginCapture(s.stream, cudaStreamCaptureModeThreadLocal));
		forward(s, sb, n_want, kv_rows, longest);
		CUDA_CHECK(cudaStreamEndCapture(s.stream, &graph));
		CUDA_CHECK(cudaGraphInstantiate(&exec, graph, 0));
		CUDA_CHECK(cudaGraphDestroy(graph));
		it = s.graphs.emplace(key, std::make_pair(exec, (int)(g_seq_launches - before))).first;
		g_seq_launches = before;
	}
	CUDA_CHECK(cudaGraphLaunch(it->second.first, s.stream));
	g_seq_launches += it->second.second;
}

} // namespace

// ---------------------------------------------------------------- C ABI

extern "C" void* calm_b200_seq_upload(const void* host, size_t size) {
	void* p = dalloc(size);
	CUDA_CHECK(cudaMemcpy(p, host, size, cudaMemcpyHostToDevice));
	return p;
}
extern "C" void calm_b200_seq_free(void* p) { cudaFree(p); }
extern "C" uint64_t calm_b200_seq_launch_count(void) { return g_seq_launches; }

extern "C" void* calm_b200_seq_prepare(const struct SeqModel* model) {
	int count = 0;
	if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) CALM_FATAL("no CUDA device available; this backend has no CPU fallback");
	Seq* sp = new Seq;
	Seq& s = *sp;
	s.m = *model;
	s.layers.assign(model->layers, model->layers + model->n_layers);
	s.m.layers = s.layers.data();
	s.pairs.reserve(s.layers.size()); // the records a pair points at are copied too
	for (SeqLayer& L : s.layers)
		if (L.type == SEQ_PAIR && L.pair) {
			s.pairs.push_back({L.pair[0], L.pair[1]});
			L.pair = s.pairs.back().data();
		}
	s.streams = s.m.block == SEQ_BLOCK_HYPER && s.m.streams > 1 ? s.m.streams : 1;
	validate(s);
	int dev = 0;
	CUDA_CHECK(cudaGetDevice(&dev));
	cudaDeviceProp prop;
	CUDA_CHECK(cudaGetDeviceProperties(&prop, dev));
	if (prop.major != 10) CALM_FATAL("device is sm_%d%d; this library is built for sm_100a only", prop.major, prop.minor);
	s.sms = prop.multiProcessorCount;
	CUDA_CHECK(cudaStreamCreate(&s.stream));
	for (cudaEvent_t& e : s.ev) CUDA_CHECK(cudaEventCreate(&e));
	for (cudaEvent_t& e : s.timer) CUDA_CHECK(cudaEventCreate(&e));
	if (const char* e = getenv("CALM_B200_SEQ_ATTN_PRODUCTS")) s.attn_products = atoi(e) != 0;
	if (const char* e = getenv("CALM_B200_SEQ_GRAPH")) s.use_graph = atoi(e) != 0;
	if (const char* e = getenv("CALM_B200_SEQ_PDL")) s.pdl = atoi(e) != 0;
	const char* tc = getenv("CALM_B200_SEQ_TC");
	s.tc = !s.m.exact && !(tc && atoi(tc) == 0);
	if (s.tc) gemm_tc_setup();

	// order of layer runs: the looped span repeated, each pass with its own state
	const SeqModel& m = s.m;
	const int times = m.loop_times > 1 ? m.loop_times : 1;
	const int ls = times > 1 ? m.loop_start : 0, le = times > 1 ? m.loop_stop : 0;
	for (int i = 0; i < ls; ++i) s.runs.push_back(RunState{i});
	for (int t = 0; t < times && le > ls; ++t)
		for (int i = ls; i < le; ++i) {
			RunState r{i};
			r.readd = t > 0 && i == ls;
			s.runs.push_back(r);
		}
	for (int i = le; i < m.n_layers; ++i) s.runs.push_back(RunState{i});

	// pages: every live token, one partly filled page per sequence
	s.n_pages = cdiv(m.max_tokens, m.page) + m.max_seqs;
	s.max_pages = s.n_pages;
	for (int p = s.n_pages - 1; p >= 0; --p) s.free_pages.push_back(p);
	s.slots.resize(m.max_seqs);
	s.table.assign((size_t)m.max_seqs * s.max_pages, 0);
	s.table_dev = (int*)dalloc(s.table.size() * sizeof(int));
	const size_t rows = (size_t)s.n_pages * m.page;
	std::function<void(RunState&, const SeqLayer&)> give = [&](RunState& r, const SeqLayer& L) { // what a run of this mixer owns
		if (L.type == SEQ_PAIR) {
			r.sub.assign(2, RunState{r.layer});
			give(r.sub[0], L.pair[0]), give(r.sub[1], L.pair[1]);
			return;
		}
		if (L.type == SEQ_LATENT) r.cache_a = (float*)dalloc(rows * L.kv_rank * sizeof(float));
		if (L.type == SEQ_WINDOW || L.type == SEQ_GQA) {
			r.cache_a = (float*)dalloc(rows * L.kv_heads * L.dim * sizeof(float));
			r.cache_b = (float*)dalloc(rows * L.kv_heads * L.vdim * sizeof(float));
		}
		if (L.type == SEQ_GQA && L.dist_bias) { // the penalty per position of distance: 2^(-8 (h+1) / heads)
			std::vector<float> sl(L.heads);
			for (int h = 0; h < L.heads; ++h) sl[h] = (float)exp2(-8.0 * (h + 1) / L.heads);
			r.slopes = (float*)dalloc(L.heads * sizeof(float));
			CUDA_CHECK(cudaMemcpy(r.slopes, sl.data(), L.heads * sizeof(float), cudaMemcpyHostToDevice));
		}
		if (L.type == SEQ_DELTA || L.type == SEQ_WINDOW || L.type == SEQ_MAMBA2) {
			r.conv_per_slot = (size_t)std::max(L.taps - 1, 0) * conv_channels(L);
			r.conv = (float*)dalloc(r.conv_per_slot * m.max_seqs * sizeof(float));
		}
		if (L.type == SEQ_DELTA) {
			r.delta_per_slot = (size_t)L.heads * L.dim * L.vdim;
			r.delta = (float*)dalloc(r.delta_per_slot * m.max_seqs * sizeof(float));
			const size_t smem = ((size_t)L.dim * L.vdim + 3 * L.dim) * sizeof(float);
			if (smem > 48 * 1024) CUDA_CHECK(cudaFuncSetAttribute(k_seq_delta_scan, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
		}
		if (L.type == SEQ_GLA || is_lin(L)) { // the scan's own layout: a value column's key channels side by side, padded to its four lanes' share
			r.delta_per_slot = (size_t)L.heads * (is_lin(L) ? lin_vs(L) : L.vdim) * gla_ldstate(L.dim);
			r.delta = (float*)dalloc(r.delta_per_slot * m.max_seqs * sizeof(float));
		}
		if (L.type == SEQ_MLSTM) {
			r.m_per_slot = L.heads;
			r.mstate = (float*)dalloc(r.m_per_slot * m.max_seqs * sizeof(float));
		}
	};
	for (RunState& r : s.runs) give(r, s.layers[r.layer]);
	gla_each([&](auto r, auto p) {
		constexpr int R = decltype(r)::value, P = decltype(p)::value;
		CUDA_CHECK(cudaFuncSetAttribute(k_seq_gla_scan<R, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gla_smem(R, P)));
	});
	CUDA_CHECK(cudaFuncSetAttribute(k_seq_attention<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
	CUDA_CHECK(cudaFuncSetAttribute(k_seq_attention<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
	// rotation tables of the grouped-query attentions: angle step per rotated pair (in double), rescaled between two wavelengths
	std::function<void(const SeqLayer&)> rot_table = [&](const SeqLayer& L) {
		if (L.type == SEQ_PAIR) {
			rot_table(L.pair[0]), rot_table(L.pair[1]);
			return;
		}
		if (L.type != SEQ_GQA || L.rot_dims < 2) return;
		const int dims = L.rot_dims, half = dims / 2;
		std::vector<double> f(half);
		float mag = 1.f;
		for (int j = 0; j < half; ++j) f[j] = pow((double)L.rot_base, -2.0 * j / dims);
		if (L.rot_factor > 0.f) {
			// the pair whose wavelength fits `t` times into the original context: pairs below `lo` keep their step, pairs above `hi`
			// turn `factor` times slower, a linear ramp between
			auto where = [&](double t) { return dims * log((double)L.rot_original / (2.0 * M_PI * t)) / (2.0 * log((double)L.rot_base)); };
			const double lo = std::max(floor(where(L.rot_fast)), 0.0), hi = std::min(ceil(where(L.rot_slow)), (double)dims - 1.0);
			for (int j = 0; j < half; ++j) {
				const double ramp = std::min(1.0, std::max(0.0, (j - lo) / std::max(hi - lo, 0.001)));
				f[j] = f[j] / L.rot_factor * ramp + f[j] * (1.0 - ramp);
			}
			mag = (float)(0.1 * log((double)L.rot_factor) + 1.0);
		}
		double* dev = (double*)dalloc(half * sizeof(double));
		CUDA_CHECK(cudaMemcpy(dev, f.data(), half * sizeof(double), cudaMemcpyHostToDevice));
		s.rot[&L] = std::make_pair(dev, mag);
	};
	for (const SeqLayer& L : s.layers) rot_table(L);
	// workspace widths
	std::function<void(const SeqLayer&)> widths = [&](const SeqLayer& L) {
		if (L.type == SEQ_PAIR) {
			widths(L.pair[0]), widths(L.pair[1]);
			if (L.w_in) s.w_proj = std::max(s.w_proj, (size_t)pair_stride(L));
			return;
		}
		if (L.ff > 0 && L.ff_kind == SEQ_FF_MOE) {
			s.max_top = std::max(s.max_top, L.top), s.max_experts = std::max(s.max_experts, L.experts + L.ident), s.w_moe_ff = std::max(s.w_moe_ff, (size_t)L.ff);
			s.w_proj = std::max(s.w_proj, (size_t)L.experts + L.ident);
			if (L.shared_ff > 0) s.w_fsh = std::max(s.w_fsh, (size_t)2 * L.shared_ff + 1 + L.experts + L.ident);
			s.w_a = std::max(s.w_a, (size_t)L.shared_ff);
		}
		if (L.type == SEQ_GQA) s.w_f = std::max(s.w_f, (size_t)L.heads * L.dim), s.w_a = std::max({s.w_a, (size_t)L.heads * L.vdim, (size_t)L.heads * L.dim * (L.scores_f32 ? 3 : 1)}); // a3 holds the queries (as value + remainder pairs when scores keep fp32 accuracy)
		if (L.type == SEQ_GLA) s.w_f = std::max({s.w_f, (size_t)L.heads * L.dim, (size_t)L.heads * L.vdim}), s.w_a = std::max({s.w_a, (size_t)L.heads * L.vdim, (size_t)L.a_rank});
		if (is_lin(L)) {
			s.w_f = std::max({s.w_f, (size_t)L.heads * L.dim, (size_t)L.heads * lin_vs(L), (size_t)L.kv_heads * L.dim});
			s.w_a = std::max(s.w_a, (size_t)L.heads * L.vdim);
			s.w_lin = std::max(s.w_lin, (size_t)2 * L.heads * L.dim + (size_t)L.heads * lin_vs(L));
		}
		s.w_proj = std::max({s.w_proj, (size_t)proj_stride(L), (size_t)2 * L.ff});
		if (L.ff > 0 && L.ff_kind == SEQ_FF_RELU2 && L.in_tail > 0) s.w_ah = std::max(s.w_ah, (size_t)L.ff);
		size_t wf = 0, wa = (size_t)L.ff;
		if (L.type == SEQ_LATENT) wf = (size_t)L.heads * L.kv_rank, wa = std::max({wa, (size_t)L.heads * L.kv_rank, (size_t)L.heads * L.dim, (size_t)L.heads * L.vdim, (size_t)L.q_rank});
		if (L.type == SEQ_DELTA) wf = std::max((size_t)L.heads * L.dim, (size_t)L.heads * L.vdim), wa = std::max({wa, (size_t)L.heads * L.vdim, (size_t)L.a_rank + L.g_rank});
		if (L.type == SEQ_WINDOW) wf = (size_t)L.heads * L.dim, wa = std::max({wa, (size_t)L.heads * L.vdim, (size_t)L.heads * L.dim});
		s.w_f = std::max(s.w_f, wf), s.w_a = std::max(s.w_a, wa);
	};
	for (const SeqLayer& L : s.layers) {
		if (L.type == SEQ_PAIR && L.ff > 0) { // the pair's own record carries the layer's feed-forward
			SeqLayer ffonly = L;
			ffonly.type = SEQ_GQA, ffonly.heads = ffonly.kv_heads = ffonly.dim = ffonly.vdim = 0, ffonly.no_gate = 1;
			widths(ffonly);
		}
		widths(L);
	}
	return sp;
}

extern "C" void calm_b200_seq_release(void* handle) {
	Seq* s = (Seq*)handle;
	if (!s) return;
	cudaStreamSynchronize(s->stream);
	drop_graphs(*s);
	std::function<void(RunState&)> drop = [&](RunState& r) {
		cudaFree(r.cache_a), cudaFree(r.cache_b), cudaFree(r.conv), cudaFree(r.delta), cudaFree(r.mstate), cudaFree(r.slopes);
		for (RunState& q : r.sub) drop(q);
	};
	for (RunState& r : s->runs) drop(r);
	cudaFree(s->lin), cudaFree(s->fsh);
	cudaFree(s->table_dev), cudaFree(s->d_tok), cudaFree(s->d_want), cudaFree(s->d_argmax), cudaFree(s->logits), cudaFree(s->hW);
	cudaFree(s->part), cudaFree(s->a3), cudaFree(s->att_kb), cudaFree(s->att_vt), cudaFree(s->att_s), cudaFree(s->att_p), cudaFree(s->x), cudaFree(s->x0), cudaFree(s->proj), cudaFree(s->hA), cudaFree(s->a1), cudaFree(s->a2), cudaFree(s->trace_buf);
	for (float* p : s->f) cudaFree(p);
	for (auto& kv : s->rot) cudaFree(kv.second.first);
	cudaFree(s->ah), cudaFree(s->mo), cudaFree(s->moe_sel), cudaFree(s->moe_wt), cudaFree(s->moe_y), cudaFree(s->moe_d), cudaFree(s->moe_x), cudaFree(s->moe_a);
	for (cudaEvent_t e : s->ev) cudaEventDestroy(e);
	for (cudaEvent_t e : s->timer) cudaEventDestroy(e);
	cudaStreamDestroy(s->stream);
	delete s;
}

extern "C" int calm_b200_seq_open(void* handle) {
	Seq& s = *(Seq*)handle;
	for (int i = 0; i < (int)s.slots.size(); ++i)
		if (!s.slots[i].open) {
			s.slots[i].open = true, s.slots[i].len = 0, s.slots[i].last_tok = -1, s.slots[i].pages.clear();
			std::function<void(RunState&)> zero = [&](RunState& r) { // a slot that is used again starts from zero state
				if (r.conv_per_slot) CUDA_CHECK(cudaMemsetAsync(r.conv + r.conv_per_slot * i, 0, r.conv_per_slot * sizeof(float), s.stream));
				if (r.delta_per_slot) CUDA_CHECK(cudaMemsetAsync(r.delta + r.delta_per_slot * i, 0, r.delta_per_slot * sizeof(float), s.stream));
				if (r.m_per_slot) CUDA_CHECK(cudaMemsetAsync(r.mstate + r.m_per_slot * i, 0, r.m_per_slot * sizeof(float), s.stream));
				for (RunState& q : r.sub) zero(q);
			};
			for (RunState& r : s.runs) zero(r);
			return i;
		}
	return -1;
}

extern "C" int calm_b200_seq_close(void* handle, int slot) {
	Seq& s = *(Seq*)handle;
	if (slot < 0 || slot >= (int)s.slots.size() || !s.slots[slot].open) return -3;
	for (int p : s.slots[slot].pages) s.free_pages.push_back(p);
	s.slots[slot].pages.clear(), s.slots[slot].open = false, s.slots[slot].len = 0;
	return 0;
}

extern "C" int calm_b200_seq_length(void* handle, int slot) {
	Seq& s = *(Seq*)handle;
	return slot >= 0 && slot < (int)s.slots.size() && s.slots[slot].open ? s.slots[slot].len : -3;
}
extern "C" int calm_b200_seq_free_pages(void* handle) { return (int)((Seq*)handle)->free_pages.size(); }

extern "C" int calm_b200_seq_step(void* handle, int n_seq, const int* slots, const int* counts, const int* tokens, int n_want, const int* want, float* logits_host) {
	Seq& s = *(Seq*)handle;
	const SeqModel& m = s.m;
	int N = 0, need = 0;
	for (int b = 0; b < n_seq; ++b) {
		const int sl = slots[b];
		if (sl < 0 || sl >= (int)s.slots.size() || !s.slots[sl].open || counts[b] < 1) return -3;
		for (int c = 0; c < b; ++c)
			if (slots[c] == sl) return -3;
		if (m.pos_table && s.slots[sl].len + counts[b] > m.max_positions) return -3; // no position row beyond the table
		need += cdiv(s.slots[sl].len + counts[b], m.page) - (int)s.slots[sl].pages.size();
		N += counts[b];
	}
	if (n_seq < 1) return -3;
	for (int i = 0; i < N; ++i)
		if (tokens[i] < 0 || tokens[i] >= m.vocab) return -3;
	for (int i = 0; i < n_want; ++i)
		if (want[i] < 0 || want[i] >= N) return -3;
	if (need > (int)s.free_pages.size()) return -2;
	reserve_tokens(s, N, n_seq, std::max(n_want, 1));

	// pages for the new tokens, then the batch description
	double kv_rows = 0; // cache rows the causal attentions read this step
	int longest = 0;    // longest sequence after this step
	s.h_meta.resize((size_t)6 * N + 4 * n_seq);
	int *tok = s.h_meta.data(), *tslot = tok + N, *tpos = tslot + N, *tfirst = tpos + N, *skip = tfirst + N, *tprev = skip + N, *sstart = tprev + N, *scount = sstart + n_seq, *spos0 = scount + n_seq,
	    *sslot = spos0 + n_seq;
	int at = 0;
	s.hb_start.resize(n_seq), s.hb_count.resize(n_seq), s.hb_pos0.resize(n_seq), s.hb_slot.resize(n_seq);
	s.n_on_products = s.tok_on_products = 0;
	for (int b = 0; b < n_seq; ++b) {
		Slot& sl = s.slots[slots[b]];
		const size_t had = sl.pages.size();
		while ((int)sl.pages.size() * m.page < sl.len + counts[b]) {
			s.table[(size_t)slots[b] * s.max_pages + sl.pages.size()] = s.free_pages.back();
			sl.pages.push_back(s.free_pages.back()), s.free_pages.pop_back();
		}
		if (sl.pages.size() > had) { // only the new entries of this slot's row travel
			const size_t o = (size_t)slots[b] * s.max_pages + had;
			CUDA_CHECK(cudaMemcpyAsync(s.table_dev + o, s.table.data() + o, (sl.pages.size() - had) * sizeof(int), cudaMemcpyHostToDevice, s.stream));
		}
		sstart[b] = at, scount[b] = counts[b], spos0[b] = sl.len, sslot[b] = slots[b];
		for (int t = 0; t < counts[b]; ++t, ++at) tprev[at] = t ? tokens[at - 1] : sl.last_tok, tok[at] = tokens[at], tslot[at] = slots[b], tpos[at] = sl.len + t, tfirst[at] = sstart[b], skip[at] = counts[b] >= kAttnGemmMin, kv_rows += sl.len + t + 1;
		s.hb_start[b] = sstart[b], s.hb_count[b] = counts[b], s.hb_pos0[b] = sl.len, s.hb_slot[b] = slots[b];
		if (counts[b] >= kAttnGemmMin) ++s.n_on_products, s.tok_on_products += counts[b];
		sl.len += counts[b], sl.last_tok = tokens[at - 1];
		longest = std::max(longest, sl.len);
	}
	CUDA_CHECK(cudaMemcpyAsync(s.d_tok, tok, N * sizeof(int), cudaMemcpyHostToDevice, s.stream));
	CUDA_CHECK(cudaMemcpyAsync(s.d_tslot, tslot, N * sizeof(int), cudaMemcpyHostToDevice, s.stream));
	CUDA_CHECK(cudaMemcpyAsync(s.d_tpos, tpos, N * sizeof(int), cudaMemcpyHostToDevice, s.stream));
	CUDA_CHECK(cudaMemcpyAsync(s.d_tfirst, tfirst, N * sizeof(int), cudaMemcpyHostToDevice, s.stream));
	CUDA_CHECK(cudaMemcpyAsync(s.d_skip, skip, N * sizeof(int), cudaMemcpyHostToDevice, s.stream));
	if (m.bigram) CUDA_CHECK(cudaMemcpyAsync(s.d_tprev, tprev, N * sizeof(int), cudaMemcpyHostToDevice, s.stream));
	CUDA_CHECK(cudaMemcpyAsync(s.d_sstart, sstart, n_seq * sizeof(int), cudaMemcpyHostToDevice, s.stream));
	CUDA_CHECK(cudaMemcpyAsync(s.d_scount, scount, n_seq * sizeof(int), cudaMemcpyHostToDevice, s.stream));
	CUDA_CHECK(cudaMemcpyAsync(s.d_spos0, spos0, n_seq * sizeof(int), cudaMemcpyHostToDevice, s.stream));
	CUDA_CHECK(cudaMemcpyAsync(s.d_sslot, sslot, n_seq * sizeof(int), cudaMemcpyHostToDevice, s.stream));
	if (n_want) CUDA_CHECK(cudaMemcpyAsync(s.d_want, want, n_want * sizeof(int), cudaMemcpyHostToDevice, s.stream));
	SeqBatch sb;
	sb.tok = s.d_tok, sb.tslot = s.d_tslot, sb.tpos = s.d_tpos, sb.tfirst = s.d_tfirst, sb.sstart = s.d_sstart, sb.scount = s.d_scount, sb.spos0 = s.d_spos0, sb.sslot = s.d_sslot;
	sb.pages = s.table_dev, sb.N = N, sb.B = n_seq, sb.max_pages = s.max_pages, sb.page = m.page;

	bool decode = s.use_graph && !s.perf && !s.trace;
	for (int b = 0; b < n_seq && decode; ++b) decode = counts[b] == 1;
	if (decode) forward_decode_graph(s, sb, n_want, kv_rows, longest);
	else forward(s, sb, n_want, kv_rows, longest);
	s.last_want = n_want, s.last_tokens = N;
	if (n_want && logits_host) CUDA_CHECK(cudaMemcpyAsync(logits_host, s.logits, (size_t)n_want * m.vocab * sizeof(float), cudaMemcpyDeviceToHost, s.stream));
	CUDA_CHECK(cudaStreamSynchronize(s.stream));
	if (int code = gemm_tc_error()) CALM_FATAL("seq: the tensor-core product pipeline stalled (code %d)", code);
	return 0;
}

extern "C" void calm_b200_seq_argmax(void* handle, int* out) {
	Seq& s = *(Seq*)handle;
	if (!s.last_want) return;
	launch_k(s, k_seq_argmax, s.last_want, 256, 0, s.logits, s.m.vocab, s.d_argmax);
	CUDA_CHECK(cudaGetLastError());
	++g_seq_launches;
	CUDA_CHECK(cudaMemcpyAsync(out, s.d_argmax, s.last_want * sizeof(int), cudaMemcpyDeviceToHost, s.stream));
	CUDA_CHECK(cudaStreamSynchronize(s.stream));
}
extern "C" const float* calm_b200_seq_device_logits(void* handle) { return ((Seq*)handle)->logits; }

extern "C" void calm_b200_seq_set_trace(void* handle, int on) { ((Seq*)handle)->trace = on != 0; }
extern "C" int calm_b200_seq_layer_runs(void* handle) { return (int)((Seq*)handle)->runs.size(); }
extern "C" void calm_b200_seq_read_trace(void* handle, int run, float* out) {
	Seq& s = *(Seq*)handle;
	if (!s.trace_buf || run < 0 || run >= (int)s.runs.size()) return;
	const size_t n = (size_t)s.last_tokens * s.m.width;
	CUDA_CHECK(cudaMemcpy(out, s.trace_buf + run * n, n * sizeof(float), cudaMemcpyDeviceToHost));
}

extern "C" void calm_b200_seq_timer_start(void* handle) {
	Seq& s = *(Seq*)handle;
	CUDA_CHECK(cudaEventRecord(s.timer[0], s.stream));
}
extern "C" float calm_b200_seq_timer_stop(void* handle) {
	Seq& s = *(Seq*)handle;
	CUDA_CHECK(cudaEventRecord(s.timer[1], s.stream));
	CUDA_CHECK(cudaEventSynchronize(s.timer[1]));
	float ms = 0;
	CUDA_CHECK(cudaEventElapsedTime(&ms, s.timer[0], s.timer[1]));
	return ms;
}
extern "C" void calm_b200_seq_set_perf(void* handle, int on) {
	Seq& s = *(Seq*)handle;
	s.perf = on != 0;
	if (on)
		for (int k = 0; k < KD_COUNT; ++k) s.kind_ms[k] = s.kind_bytes[k] = s.kind_flops[k] = 0, s.kind_launches[k] = 0;
}
extern "C" int calm_b200_seq_perf_stats(void* handle, int kind, char* name, int name_cap, double* ms_total, double* bytes_total, double* flops_total, long* launches) {
	Seq& s = *(Seq*)handle;
	if (kind < 0 || kind >= KD_COUNT) return 0;
	snprintf(name, name_cap, "%s", kKindNames[kind]);
	*ms_total = s.kind_ms[kind], *bytes_total = s.kind_bytes[kind], *flops_total = s.kind_flops[kind], *launches = s.kind_launches[kind];
	return 1;
}
