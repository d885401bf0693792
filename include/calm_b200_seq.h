/*
 * calm_b200_seq.h -- C ABI of libcalm_b200_seq.so: layer-list models served to MANY sequences at once.
 *
 * The calm boundary (calm_b200.h) serves one sequence of a Llama-shaped model per process.  This boundary serves models
 * whose layers are given as a list (each entry names a token mixer and a feed-forward) to a batch of sequences, each with
 * its own cache and recurrent state, and follows the same protocol: the host parses the container, uploads every tensor
 * with calm_b200_seq_upload(), binds the device pointers in the records below and calls calm_b200_seq_prepare().  After
 * that, sequences are opened, stepped (any number of new tokens per sequence and step: a prompt, a portion of one, or a
 * single decoded token) and closed.  Errors that are the caller's (no slot, no page left, a closed slot) come back as
 * negative return codes; CUDA failures print one line and abort(), as everywhere in this library.  No CPU fallback.
 *
 * Mixers (SeqLayer.type):
 *   SEQ_LATENT  latent attention: queries and keys/values go through low-rank latents, only the normalised key/value
 *               latent is cached; causal softmax; a sigmoid gate per head on the output.
 *   SEQ_DELTA   gated delta rule with one decay per head and key channel: short causal convolutions + SiLU on q, k, v,
 *               unit-norm q and k, a [dim x vdim] fp32 state per head carried from token to token.
 *   SEQ_WINDOW  grouped-query attention behind short causal convolutions, unweighted RMS norm on q and k, a sliding
 *               window of `window` positions and a learned per-head sink in the softmax denominator.
 *   SEQ_GQA     grouped-query attention with biased projections, one RMS norm over the whole query (and key) projection,
 *               rotation of the first rot_dims channels of every head (pairs i, i + rot_dims/2; frequencies optionally
 *               rescaled between two wavelengths), a sliding window that also keeps the first keep_first positions, and a
 *               sigmoid gate on every output channel.
 *   SEQ_GLA     gated linear attention: a [dim x vdim] fp32 state per head, S <- diag(a) S + k v^T, o = S^T q, with a decay
 *               a = sigmoid(.)^(1/tau) per key channel from a low-rank projection; per-head RMS norm and a SiLU gate on the output.
 *               Options of SEQ_GQA: `chunk` (a query sees only the keys of its own block of `chunk` positions, counted from position 0),
 *               `dist_bias` (score -= 2^(-8 (h+1) / heads) * distance), `add_one` (one added to the softmax denominator),
 *               `v_norm` (every value head divided by its root mean square before it is cached), `no_gate`.
 *   SEQ_MLSTM   matrix memory with exponential gating: per head a [dim x vdim] fp32 state S, a normaliser n and a running maximum m
 *               (zero at the start) of the log gates; log input gate cap tanh(./cap), log forget gate logsigmoid(cap tanh(./cap));
 *               o = S^T q / (max(|n.q|, exp(-m)) + 1e-6); per-head RMS, a weight per output channel, a sigmoid gate.
 *   SEQ_HGRN2   linear attention whose forget gate f = l + (1 - l) sigmoid(.) per key channel (lower bound l) also writes:
 *               S <- diag(f) S + (1 - f) v^T, o = S^T silu(q); per-head RMS norm with a weight shared by the heads.
 *   SEQ_MAMBA2  state-space mixer: one input product [z | x | B | C | dt], a short causal convolution with bias and SiLU over x, B, C,
 *               dt = softplus(dt + dt_bias), per head S <- exp(-exp(A_log) dt) S + dt B x^T ([state x vdim]), y = S^T C + D x,
 *               y silu(z), RMS norm in norm_groups equal parts with a weight per channel.  kv_heads = groups of B / C, dim = state.
 *   SEQ_PAIR    two mixers side by side on the same input (`pair` points at two SeqLayer records, their feed-forward unused):
 *               pair_scale[0] * first + pair_scale[1] * second.  When the pair's own record has w_in (and b_in), it holds both mixers'
 *               input rows as one matrix -- the first's, zero rows up to a multiple of 8, the second's -- for one product; the two
 *               records then have no w_in of their own (served for SEQ_GQA and SEQ_GLA).
 * Norms (SeqModel.norm_kind): Dynamic Tanh (tanh(alpha x) w + b), or RMS (x / sqrt(mean x^2 + eps) * (w + norm_offset)).
 * Blocks (SeqModel.block): serial -- norm, mixer, norm, residual add, then the same around the feed-forward; parallel -- one
 * norm whose output both the mixer and the feed-forward read, x <- x + (mixer + feed-forward); hyper -- the residual is `streams`
 * copies x_1 .. x_S; sublayer q reads u = sum_s in[s] x_s, y = sublayer(norm(u)), and x_t <- sum_s mix[s][t] x_s + out[t] y for all
 * t at once; the model's output is the sum of the streams.  (One stream with in = out = mix = 1 is the plain pre-norm residual.)
 * A norm whose weight is a single number for all columns: SeqModel.norm_scalar.  Learned positions: SeqModel.pos_table.
 * Feed-forward (SeqLayer.ff_kind): clamped gated unit, down(relu(up)^2), or a routed mixture of SiLU-gated experts (the `top`
 * highest router scores, mixed by a softmax restricted to those scores; or, route_mode 1, a softmax over all router outputs,
 * the choice made on score + correction, the weights score * route_scale, not renormalised).  The last `ident` router outputs are
 * identity experts (output = input); a shared unit of the same form (shared_ff) runs for every token and is added.
 * A span of layers can be run several times in a row with the same weights (loop_*), each pass with its own state.
 *
 * Post-norm blocks (SEQ_BLOCK_POST): a sublayer reads the residual stream itself (rounded to the activation type) and its output
 * comes back through the model's RMS norm, x <- x + norm1(mixer(x)), then x <- x + norm2(feed-forward(x)).  Any mixer of the list
 * runs in them, pairs included.
 * Options of SEQ_GQA added for them: `qk_per_head` (the query / key RMS norm runs over each head's `dim` channels with one weight
 * vector [dim] shared by the heads), `gate_per_head` (one sigmoid gate per head: `heads` gate rows in w_in), `b_o` (a bias of the
 * output projection), `scores_f32` (scores and softmax weights keep fp32 accuracy also where a prompt's attention runs as tensor-core products).
 * Feed-forward SEQ_FF_GATED: down(act(gate) * up) with act = SiLU or the tanh form of GELU (ff_act).
 * Routed experts, further options: `expert_act` 1 -- an expert (and the shared unit) is down(relu(up)^2), without gate rows;
 * route_mode 2 -- scores are sigmoid(router output), the `top` highest are taken, the weights are those scores times route_scale,
 * not renormalised; `weight_input` -- the weight multiplies the expert's input instead of its output; `shared_gate` -- the shared
 * unit's output is multiplied by sigmoid(one more row of its first product), one number per token.
 * Embedding: SeqModel.bigram adds row (previous token * mul_prev + token * mul_cur) mod buckets of a second table (row `buckets`
 * for a sequence's first token); the previous token is kept with the sequence's slot.  SeqModel.logit_scale multiplies the logits.
 */
#ifndef CALM_B200_SEQ_H
#define CALM_B200_SEQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum SeqMixer { SEQ_LATENT = 0, SEQ_DELTA = 1, SEQ_WINDOW = 2, SEQ_GQA = 3, SEQ_GLA = 4, SEQ_MLSTM = 5, SEQ_HGRN2 = 6, SEQ_MAMBA2 = 7, SEQ_PAIR = 8 };
enum SeqNormKind { SEQ_NORM_DYT = 0, SEQ_NORM_RMS = 1 };
enum SeqBlock { SEQ_BLOCK_SERIAL = 0, SEQ_BLOCK_PARALLEL = 1, SEQ_BLOCK_HYPER = 2, SEQ_BLOCK_POST = 3 };
enum SeqFfKind { SEQ_FF_CLAMPED = 0, SEQ_FF_RELU2 = 1, SEQ_FF_MOE = 2, SEQ_FF_GATED = 3 };
enum SeqFfAct { SEQ_ACT_SILU = 0, SEQ_ACT_GELU_TANH = 1 };

/* a norm: bf16 weight[n]; Dynamic Tanh also bf16 bias[n], bf16 alpha[1] (device pointers; NULL for an RMS norm) */
struct SeqNorm {
	const void* w;
	const void* b;
	const void* alpha;
};

/* hyper-connection of one sublayer: bf16 in[streams], out[streams], mix[streams][streams] (indexed [from][to]) */
struct SeqHyper {
	const void* in;
	const void* out;
	const void* mix;
};

/* One layer.  All matrices are bf16, row-major (out, in), device pointers.  w_in is the layer's input projections
 * stacked by rows in the order given per mixer below. */
struct SeqLayer {
	int type;            /* enum SeqMixer */
	int heads, kv_heads; /* SEQ_LATENT: kv_heads unused */
	int dim, vdim;       /* per-head query/key width and value width */
	int q_rank, kv_rank; /* SEQ_LATENT */
	int taps;            /* SEQ_DELTA / SEQ_WINDOW: convolution taps (1 = none) */
	int window;          /* SEQ_WINDOW: positions seen, the current one included; <= 0: unbounded */
	int a_rank, g_rank;  /* SEQ_DELTA: inner widths of the decay and gate projections */
	int ff;              /* feed-forward width, 0 = no feed-forward */
	float scale;         /* score scale of the attentions */
	float limit;         /* clamp of the feed-forward */
	struct SeqNorm norm1, norm1b, norm2, norm2b;
	/* SEQ_LATENT: rows [dq | dkv | g];  SEQ_DELTA: [q | k | v | b | a1 | g1];  SEQ_WINDOW: [q | k | v];
	 * SEQ_GQA: [q | k | v | g] (no_gate: [q | k | v]);  SEQ_GLA: [q | k | v | g | a1];  SEQ_MLSTM: [q | k | v | g | i | f];
	 * SEQ_HGRN2: [q | f | v];  SEQ_MAMBA2: [z | x | B | C | dt] */
	const void* w_in;
	const void* w_o;       /* (width, heads*vdim) */
	/* SEQ_LATENT */
	const void* dq_norm;   /* bf16 [q_rank] */
	const void* dkv_norm;  /* bf16 [kv_rank] */
	const void* w_uq;      /* (heads*dim, q_rank) */
	const void* w_ukT;     /* per head the TRANSPOSED key up-projection: [heads][kv_rank][dim] */
	const void* w_uv;      /* (heads*vdim, kv_rank) */
	/* SEQ_DELTA / SEQ_WINDOW */
	const void* conv;      /* bf16 [channels of q|k|v][taps] */
	/* SEQ_DELTA */
	const void* w_a2;      /* (heads*dim, a_rank) */
	const void* w_g2;      /* (heads*vdim, g_rank) */
	const void* a_log;     /* bf16 [heads] */
	const void* dt_bias;   /* bf16 [heads*dim] */
	const void* out_norm;  /* bf16 [vdim] */
	/* SEQ_WINDOW */
	const void* sink;      /* bf16 [heads] or NULL */
	/* feed-forward */
	const void* w_gate_up; /* rows [gate | up]: (2*ff, width); SEQ_FF_RELU2: up only (ff, width); SEQ_FF_MOE: [experts](2*ff, width) */
	const void* w_down;    /* (width, ff); SEQ_FF_MOE: [experts](width, ff) */
	/* SEQ_GQA / SEQ_GLA */
	const void* b_in;      /* bf16 bias of the stacked input projection (rows of w_in), or NULL */
	const void* q_norm;    /* SEQ_GQA: bf16 [heads*dim], weight of the RMS norm over the whole query projection, or NULL */
	const void* k_norm;    /* SEQ_GQA: bf16 [kv_heads*dim] */
	const void* b_a2;      /* SEQ_GLA: bf16 [heads*dim], bias of the decay projection */
	int keep_first;        /* SEQ_GQA: the first positions every query keeps seeing (with `window`) */
	int rot_dims;          /* SEQ_GQA: rotated channels per head (even, <= dim; 0: none) */
	float rot_base;
	float rot_factor;      /* frequency rescaling between two wavelengths; <= 0: none */
	float rot_original, rot_fast, rot_slow;
	float tau;             /* SEQ_GLA: decay = sigmoid(.)^(1/tau) */
	int ff_kind;           /* enum SeqFfKind; ff is the width of one expert for SEQ_FF_MOE */
	int experts, top;      /* SEQ_FF_MOE */
	const void* w_router;  /* (experts, width) */
	const void* b_router;  /* bf16 [experts] or NULL */
	/* parallel blocks: the feed-forward reads the same normed input as the mixer, so its first rows can ride in the mixer's input
	 * product.  in_tail rows appended to w_in (and b_in): SEQ_FF_MOE: the router's `experts` rows (w_router / b_router unused);
	 * SEQ_FF_RELU2: the `ff` rows of the up projection (w_gate_up unused); 0: the feed-forward runs its own first product */
	int in_tail;
	/* SEQ_GQA options */
	int chunk;             /* > 0: a query at position p sees keys from floor(p / chunk) * chunk on */
	int dist_bias;         /* 1: score -= 2^(-8 (h+1) / heads) * (query position - key position) */
	int add_one;           /* 1: one is added to the softmax denominator */
	int v_norm;            /* 1: each value head is divided by its root mean square (eps, no weight) before it is cached */
	int no_gate;           /* 1: no output gate (and no gate rows in w_in) */
	/* SEQ_MLSTM */
	float gate_cap;        /* soft cap of both gate pre-activations */
	/* SEQ_HGRN2 */
	const void* lower;     /* bf16 [heads*dim]: lower bound of the forget gate */
	/* SEQ_MAMBA2 (also a_log [heads], dt_bias [heads], conv [channels][taps], out_norm [heads*vdim]) */
	const void* conv_b;    /* bf16 [channels]: bias of the convolution, or NULL */
	const void* skip_d;    /* bf16 [heads]: y += D x */
	int norm_groups;       /* the output norm runs over heads*vdim / norm_groups columns at a time */
	/* SEQ_PAIR */
	const struct SeqLayer* pair; /* two records */
	float pair_scale[2];
	/* SEQ_BLOCK_HYPER */
	struct SeqHyper hc1, hc2;
	/* SEQ_FF_MOE extras */
	int route_mode;        /* 0: softmax over the chosen logits; 1: softmax over all, choice on score + correction, weight = score * route_scale;
	                          2: score = sigmoid(output), choice on score, weight = score * route_scale */
	int ident;             /* identity experts: router outputs experts .. experts + ident - 1 (w_router has experts + ident rows) */
	float route_scale;
	const void* correction; /* bf16 [experts + ident] or NULL */
	int shared_ff;         /* width of the shared unit, 0: none */
	const void* w_sh_gate_up; /* (2*shared_ff, width) rows [gate | up]; with w_router == NULL the router's experts + ident rows follow them (one product) */
	const void* w_sh_down;    /* (width, shared_ff) */
	/* SEQ_GQA, further options */
	int qk_per_head;       /* 1: q_norm / k_norm are bf16 [dim], the RMS norm runs over each head's channels */
	int gate_per_head;     /* 1: the gate rows of w_in are `heads` rows, one sigmoid gate per head */
	const void* b_o;       /* bf16 [width]: bias of the output projection, or NULL (any mixer) */
	int scores_f32;        /* 1: scores and softmax weights keep fp32 accuracy also where prompts run as tensor-core products: queries, keys and probabilities
	                          travel as bf16 pairs (value + remainder of the rounding), values as bf16 */
	/* SEQ_FF_GATED */
	int ff_act;            /* enum SeqFfAct: activation of the gate rows (w_gate_up rows [gate | up]) */
	/* SEQ_FF_MOE, further options */
	int expert_act;        /* 0: an expert is down(silu(gate) * up), rows [gate | up]; 1: down(relu(up)^2), w_gate_up = [experts](ff, width), the shared unit alike */
	int weight_input;      /* 1: a choice's weight multiplies the expert's input */
	int shared_gate;       /* 1: w_sh_gate_up has one more row behind the unit's first rows (before the router's): the shared output is multiplied by its sigmoid */
};

struct SeqModel {
	int vocab, width, n_layers;
	int loop_start, loop_stop, loop_times; /* layers [start, stop) run `times` times; times <= 1: no loop */
	float eps;
	int exact;       /* 1: every product in true fp32 (SIMT), 0: bf16 tensor-core products with fp32 accumulation */
	int max_tokens;  /* tokens that live sequences hold at any time: sizes the paged cache */
	int max_seqs;    /* sequence slots */
	int page;        /* tokens per cache page */
	const void* embed;  /* bf16 (vocab, width) */
	const void* head;   /* bf16 (vocab, width) */
	struct SeqNorm final_norm;
	const struct SeqLayer* layers;
	int norm_kind;      /* enum SeqNormKind */
	float norm_offset;  /* SEQ_NORM_RMS: added to the stored weight (1 when the checkpoint keeps weights as offsets from one) */
	int block;          /* enum SeqBlock */
	float embed_scale;  /* factor on the embedding rows (0 is read as 1) */
	int streams;        /* SEQ_BLOCK_HYPER: copies of the residual stream (0 is read as 1) */
	int norm_scalar;    /* 1: every norm weight of the model is one number (bf16 [1]) for all columns */
	const void* pos_table; /* bf16 (max_positions, width): learned position rows added to the embedding, or NULL */
	int max_positions;  /* rows of pos_table: no sequence grows beyond */
	const void* bigram; /* bf16 (bigram_buckets + 1, width): rows added to the embedding, picked by a hash of (previous token, token); or NULL */
	int bigram_buckets, bigram_mul_prev, bigram_mul_cur;
	float logit_scale;  /* factor on the logits (0 is read as 1) */
};

/* cudaMalloc + copy, like upload_cuda */
void* calm_b200_seq_upload(const void* host, size_t size);
void calm_b200_seq_free(void* device_ptr);

/* Validate, allocate the page pool and per-slot state; returns an opaque handle (NULL never: failures abort). */
void* calm_b200_seq_prepare(const struct SeqModel* model);
void calm_b200_seq_release(void* handle);

/* Sequence slots.  open: a free slot with empty cache and zero state, or -1.  close: pages and slot go back. */
int calm_b200_seq_open(void* handle);
int calm_b200_seq_close(void* handle, int slot);
int calm_b200_seq_length(void* handle, int slot);
int calm_b200_seq_free_pages(void* handle);

/* One step over a batch: sequence i (slot slots[i]) is fed counts[i] new tokens, packed back to back in `tokens`.
 * `want` lists n_want packed token indices (ascending or not) whose logits are computed; they stay on the device and,
 * when logits_host != NULL, are copied there as float[n_want][vocab].  Returns 0, or -2 when the page pool is
 * exhausted, -3 for a bad slot / count (nothing has run then). */
int calm_b200_seq_step(void* handle, int n_seq, const int* slots, const int* counts, const int* tokens, int n_want, const int* want,
                       float* logits_host);

/* argmax (lowest index wins ties) of each row of the last step's logits -> out[n_want] */
void calm_b200_seq_argmax(void* handle, int* out);
/* device pointer of the last step's logits, float[n_want][vocab] */
const float* calm_b200_seq_device_logits(void* handle);

/* (tests) residual stream of the last step after layer run `run`: float[n_tokens][width]; only recorded when
 * calm_b200_seq_set_trace(handle, 1) was called before the step */
void calm_b200_seq_set_trace(void* handle, int on);
int calm_b200_seq_layer_runs(void* handle);
void calm_b200_seq_read_trace(void* handle, int run, float* out);

uint64_t calm_b200_seq_launch_count(void);
void calm_b200_seq_timer_start(void* handle);
float calm_b200_seq_timer_stop(void* handle);
/* per-kernel-kind device time of the steps since set_perf(handle, 1): events around every launch (slow; for the bench's
 * roofline table only).  stats: returns 0 past the last kind. */
void calm_b200_seq_set_perf(void* handle, int on);
int calm_b200_seq_perf_stats(void* handle, int kind, char* name, int name_cap, double* ms_total, double* bytes_total, double* flops_total, long* launches);

#ifdef __cplusplus
}
#endif

#endif /* CALM_B200_SEQ_H */
