"""What every layer and setting is, and what its fields do: one catalogue that the
editor's hovers and completions (`bux_b200.lang.lsp`) and the generated reference pages
(`bux_b200.lang.reference`) both read.

`SUMMARY[tag]` is one sentence on the thing called `tag` in a ``.bux`` file;
`FIELDS[tag][field]` is a note on one of its fields. A note written under a family key of
`FAMILIES` (``"attention"``, ``"recurrent"``, ...) holds for every tag of the family, so a
field shared by eight mixers is written once. The text is Markdown. A tag or field
without an entry is still listed by the reference with its type and default: the
catalogue adds prose, the schema stays the source of names, types and defaults.
"""

from __future__ import annotations

SUMMARY = {
    # ---- layers
    "embed": "Token embedding: ids to rows of a `vocab_size x d_model` table; the model's first layer.",
    "head": "Language-model head: the stream to logits over the vocabulary; the layer the loss reads.",
    "rmsnorm": "RMS normalisation over the channel axis with a learned gain.",
    "layernorm": "Layer normalisation (mean and variance) over the channel axis.",
    "dyt": "Dynamic tanh: `tanh(alpha * x)` with a learned scalar `alpha` and gain, a normaliser without statistics.",
    "mlp": "Two-projection feed-forward block: up, activation, down.",
    "gated_mlp": "Gated feed-forward block (SwiGLU and relatives): `down(act(gate(x)) * up(x))`.",
    "moe": "Mixture of experts: a router picks `top_k` of `num_experts` feed-forward experts per token.",
    "gqa": "Softmax attention with grouped key/value heads (MHA when `num_kv_heads == num_heads`, MQA when 1).",
    "mla": "Multi-head latent attention: keys and values are expanded from one low-rank latent per token.",
    "csa": "Compressed sparse attention: a sliding window plus latents that each summarise `compress_ratio` tokens, in one softmax.",
    "deltanet": "Linear attention with the delta rule: the state is corrected toward each new key/value pair.",
    "gdn": "Gated DeltaNet: the delta rule with a per-head scalar decay of the state.",
    "gdn2": "Gated DeltaNet-2: per-channel decay from a low-rank gate, optional negative eigenvalues.",
    "kda": "Kimi delta attention: the delta rule with a per-channel decay.",
    "gla": "Gated linear attention: a decayed outer-product state with a per-channel gate.",
    "lightning": "Lightning attention: linear attention with a fixed per-head decay that depends on the layer's depth.",
    "rwkv7": "RWKV-7 time mixing: a generalised delta rule with learned in-context learning rates.",
    "mamba": "Selective state-space layer (Mamba): input-dependent step size, diagonal state.",
    "mamba2": "Mamba-2: a scalar-decay state-space layer with heads, a chunked scan.",
    "conv": "Causal depthwise convolution over the tokens.",
    "short_conv": "A short causal depthwise convolution with a residual input, as the mixers use before their recurrences.",
    "linear": "A dense projection to `features` channels.",
    "act": "An activation function applied elementwise; written by its name (`swish`, `gelu`, ...).",
    "scale": "Multiplication by a learned scalar (or one weight per channel).",
    "dropout": "Dropout on the stream; identity in evaluation.",
    "value_embed": "A second embedding of the tokens that attention layers can add to their values through a port.",
    "nextn": "Multi-token-prediction input: joins the stream with the embedding of the next token.",
    "engram": "N-gram memory: hashed n-grams of the tokens index a table whose rows are gated into the stream.",
    "doc_copy": "Copy head over the document: scores earlier positions whose context matches and adds their next tokens' logits.",
    "merge": "Folds the residual algebra's streams back into one (inserted by the compiler before a head).",
    # ---- sub-configs
    "rope": "Rotary position embedding of queries and keys.",
    "pi": "Position interpolation: positions divided by `factor`.",
    "llama3": "Llama-3 frequency scaling: low frequencies slowed by `factor`, high ones kept, a smooth band between.",
    "yarn": "YaRN frequency scaling with an attention temperature.",
    "relbias": "A learned relative-position bias on the attention logits, low-rank over the distance.",
    "indexer": "Lightning indexer for sparse attention: a small scorer picks the keys (or blocks) each query attends.",
    "copy_pointer": "A pointer over the context whose copy distribution is mixed into the head's.",
    "hc": "Hyper-connections: the residual stream widened to `expansion` copies with learned read/write weights.",
    "mhc": "Manifold-constrained hyper-connections: hyper-connections whose mixing matrix is doubly stochastic (Sinkhorn).",
    "gr": "Gated residual: a low-rank gate decides how much of each branch enters the stream.",
    "attnres": "Attention residuals: each block reads a softmax-weighted mix of earlier blocks' outputs.",
    "msar": "Multi-scale attention residuals: attention residuals over pooled histories of several sizes.",
    "vpgate": "Variance-preserving gate on each branch's contribution.",
    "normal": "Normal initialisation with a fixed standard deviation, per role.",
    "fan_in": "Variance-scaling initialisation by the fan-in.",
    "fan_out": "Variance-scaling initialisation by the fan-out.",
    "fan_avg": "Variance-scaling initialisation by the mean of fan-in and fan-out.",
    "zeros": "Zero initialisation for the roles it names.",
    # ---- training
    "adamw": "AdamW with decoupled weight decay.",
    "muon": "Muon: momentum orthogonalised by Newton-Schulz for matrices, AdamW for everything else.",
    "normuon": "NorMuon: Muon with a per-row second-moment normalisation after the orthogonalisation.",
    "ema": "An average of the weights over the tail of the run, which the run ends on.",
    "constant": "Constant learning rate after a linear warm-up.",
    "cosine": "Cosine decay to `final` after a linear warm-up.",
    "linear_decay": "Linear decay to `final` after a linear warm-up.",
    "wsd": "Warm-up, stable, decay: constant, then a cool-down over the last `decay` share of the steps.",
    "power": "Power-law decay `a * step^-b` with a cool-down.",
    "multistep": "Piecewise-constant rate multiplied by `factor` at each step of `at`.",
    "piecewise": "A schedule given as pieces, each moving the rate to a value by a step.",
    "piece": "One piece of a `piecewise` schedule.",
    "text": "Documents from a text column of parquet or JSON-lines files.",
    "chat": "Conversations rendered by a chat template; the loss is masked to the roles trained on.",
    "tokens": "Pre-tokenised ids in flat binary files.",
    "synthetic": "Random tokens of the model's vocabulary: for smoke tests and benchmarks.",
    "tokenizer": "The tokenizer that turns documents into ids.",
    "concat": "Packing by concatenation: documents end to end, cut at row boundaries.",
    "greedy": "Greedy packing: whole documents in arrival order, a new row when the next one does not fit.",
    "best_fit": "Best-fit packing: each document goes to the fullest row that still has room.",
    "phase": "A curriculum phase: from step `at` on, other data, sequence length, batch or RoPE settings.",
    "ramp": "A batch-size ramp over the first steps.",
    "loss": "Terms added to the first head's cross-entropy: z-loss, the multi-token-prediction heads, prefix-token prediction.",
    "prefix": "Prefix-token prediction: beside each target the head also predicts the token whose bytes are the target's longest proper prefix in the vocabulary; its weight is held, then falls to zero.",
    "eval": "A periodic evaluation on held-out data.",
    "checkpoint": "Periodic checkpoints of the model and optimizer state.",
    "log": "How often metrics are logged and which trackers receive them.",
    "observe": "Periodic statistics of the forward pass: stream norms per branch, router loads, attention samples.",
    "profile": "A profiler capture over a window of steps.",
    "precision": "Compute dtype and the formats of the matrix multiplications.",
    "roles": "Per-role matmul formats (which projections run in MXFP8 or NVFP4).",
    "switch": "A change of the quantised passes late in training.",
    "mesh": "How many GPUs each parallel axis spans; the product is the job's size.",
    "layout": "Which mesh axis shards which logical axis of the tensors.",
    "methods": "Algorithm choices that change speed and memory, not the arithmetic of the run.",
    "remat": "What the backward recomputes instead of keeping from the forward.",
    "compiler": "Options for the step's build: presets and free-form flags.",
    "search": "A hyper-parameter search over the file's dimensions.",
    "random": "Random search.", "halton": "Halton low-discrepancy sequence.", "sobol": "Sobol low-discrepancy sequence.",
    "tpe": "Tree-structured Parzen estimator.", "gp": "Gaussian-process Bayesian optimisation (Matern 5/2).",
    "halving": "Successive halving / Hyperband: many short trials, the best continue.",
    "uniform": "A real dimension, uniform on `[low, high]`.",
    "log_uniform": "A real dimension, uniform in the logarithm.",
    "int_uniform": "An integer dimension on `[low, high]`.",
    "choice": "A dimension over listed options.",
    "wandb": "Weights & Biases tracker.", "tensorboard": "TensorBoard tracker.",
}

# tags that share field notes
FAMILIES = {
    "attention": ("gqa", "mla", "csa"),
    "recurrent": ("deltanet", "gdn", "gdn2", "kda", "gla", "lightning", "rwkv7"),
    "norm": ("rmsnorm", "layernorm"),
    "mlp": ("mlp", "gated_mlp"),
    "muon": ("muon", "normuon"),
    "schedule": ("constant", "cosine", "linear_decay", "wsd", "power", "multistep", "piecewise"),
    "packing": ("concat", "greedy", "best_fit"),
    "hc": ("hc", "mhc"),
    "fan": ("fan_in", "fan_out", "fan_avg"),
    "init": ("normal", "fan_in", "fan_out", "fan_avg", "zeros"),
    "documents": ("text", "chat"),
}

FIELDS = {
    "attention": {
        "num_heads": "Query heads.",
        "head_dim": "Channels per head; `none` means `width // num_heads`.",
        "sliding_window_size": "Each query sees at most this many most recent keys; `none` is full causal attention.",
        "softcap": "Logits pass through `cap * tanh(x / cap)` before the softmax.",
        "sinks": "One learned logit per head joins every softmax row and takes probability without a value.",
        "qk_norm": "A norm applied to queries and keys per head before RoPE.",
        "scale": "Logit scale; `none` is `head_dim ** -0.5`.",
        "log_scale": "Scales the logits by the logarithm of the position (length extrapolation).",
        "log_scale_floor": "The position below which `log_scale` leaves the logits alone.",
        "gated": "An output gate computed from the layer's input multiplies the attention output.",
        "gate_per_head": "One gate value per head instead of per channel.",
        "gate_activation": "The gate's squashing function.",
        "gate_head_bias": "A learned bias per head inside the gate.",
        "gate_input_rank": "The gate reads a low-rank projection of the input of this rank.",
        "gate_output_rank": "The gate is expanded from this rank.",
        "gate_cross_head": "The gate mixes information across heads.",
        "output_norm": "A norm on the heads' outputs before the output projection.",
        "attention_dropout": "Dropout on the attention probabilities.",
        "output_dropout": "Dropout on the layer's output.",
        "relative_bias": "A learned bias on the logits as a function of the query-key distance.",
        "indexer": "Makes the layer sparse: only the keys the indexer picks are attended.",
        "rope": "Rotary embedding of queries and keys; `none` for no positions.",
    },
    "gqa": {
        "num_kv_heads": "Key/value heads; each serves `num_heads // num_kv_heads` query heads.",
        "v_head_dim": "Channels of a value head when it differs from `head_dim`.",
        "bias": "Biases on the q, k and v projections.", "output_bias": "A bias on the output projection.",
        "fused_qkv": "One projection for q, k and v, split afterwards: the same function, held as one matrix.",
        "qk_norm_all_heads": "`qk_norm` normalises over all heads' channels at once.",
        "power_scale": "Temperature that grows as a power of the context length.",
        "power_scale_length": "The length at which `power_scale` equals one.",
        "kv_conv_size": "A short causal convolution on keys and values before attention.",
        "value_residual": "How the first layer's values (the `v` port) are mixed into this layer's: `fixed` halves, `learned` weights, or a `convex` learned blend.",
        "exclusive": "A query does not attend to its own position; `learned` gives the diagonal a learned logit instead.",
        "value_embed_gate": "Gate the value embedding added through the `ve` port.",
        "k_eq_v": "Keys and values share one projection.",
        "differential": "Differential attention: the difference of two softmax maps.",
        "paired": "Heads are paired and share their attention map.",
        "mimetic_vo": "Initialise V and O so that their product starts near a scaled identity.",
        "mimetic_noise": "Noise added to the mimetic initialisation.",
    },
    "mla": {
        "q_lora_rank": "Rank of the query's low-rank projection; `none` for a full one.",
        "kv_lora_rank": "Width of the per-token latent that keys and values are expanded from.",
        "qk_nope_head_dim": "Per-head channels of q and k that carry no position.",
        "qk_rope_head_dim": "Per-head channels of q and k that RoPE rotates (one shared key head).",
        "v_head_dim": "Channels of a value head.",
    },
    "csa": {
        "compress_ratio": "Tokens summarised by one compressed latent.",
        "q_lora_rank": "Rank of the query's low-rank projection.", "o_lora_rank": "Rank of the grouped output projection.",
        "o_groups": "Head groups of the output projection.", "latent_norm": "Norm on the compressed latents.",
    },
    "recurrent": {
        "num_heads": "Heads of keys and queries.", "head_dim": "Channels per key head.",
        "num_v_heads": "Value heads when they differ from `num_heads`.", "v_head_dim": "Channels per value head.",
        "conv_size": "Taps of the short causal convolutions before the recurrence; `none` for none.",
        "output_gate": "A gate from the input multiplies the normalised output.",
        "norm_eps": "Epsilon of the per-head output norm.",
        "gate_rank": "Rank of the low-rank projection that makes the decay gate.",
        "output_gate_rank": "Rank of the output gate's projection.",
        "gate_lower_bound": "Smallest decay the gate can produce.",
        "negative_eigenvalues": "Let the state transition have eigenvalues in (-1, 1) instead of (0, 1).",
    },
    "rwkv7": {"decay_rank": "Rank of the decay's projection.", "a_rank": "Rank of the in-context learning-rate projection.",
              "v_rank": "Rank of the value-residual projection."},
    "mamba": {"state_size": "State channels per input channel.", "expand": "Inner width as a multiple of the stream's.",
              "conv_size": "Taps of the causal convolution.", "dt_min": "Smallest initial step size.",
              "dt_max": "Largest initial step size.", "dt_rank": "Rank of the step-size projection; `none` is `width / 16`."},
    "mamba2": {"state_size": "State channels per head.", "expand": "Inner width as a multiple of the stream's.",
               "conv_size": "Taps of the causal convolution.", "head_dim": "Channels per head.",
               "num_heads": "Heads; `none` derives them from `head_dim`.", "num_groups": "Groups that share B and C.",
               "dt_min": "Smallest initial step size.", "dt_max": "Largest initial step size."},
    "norm": {
        "eps": "Added to the variance before the square root.", "affine": "Learn a gain per channel.",
        "bias": "Learn a bias per channel.", "zero_centered": "Store the gain as `1 + w` with `w` initialised to zero.",
        "gain_init": "Initial gain.", "scale_input": "Multiply by the gain before normalising, `norm(w * x)`, instead of after.",
    },
    "mlp": {
        "intermediate_size": "Hidden width.", "activation": "The nonlinearity (of the gate, for `gated_mlp`).",
        "dropout": "Dropout on the hidden activations.", "bias": "Biases on the projections.",
        "limit": "Clamp the hidden pre-activations to `[-limit, limit]`.",
        "up_softcap": "Soft cap on the up projection.", "up_offset": "Constant added to the up projection (gpt-oss adds 1).",
    },
    "moe": {
        "num_experts": "Routed experts.", "top_k": "Experts each token is sent to.",
        "expert": "The feed-forward block every expert is.",
        "num_shared_experts": "Experts every token also passes through.",
        "shared_expert": "The shared experts' block when it differs from `expert`.",
        "shared_expert_gate": "A sigmoid gate on the shared experts' output.",
        "router": "How logits become weights: `softmax` over the picks, `sigmoid` per expert, ...",
        "router_bias": "A learned bias on the router's logits.", "router_logit_scale": "Multiplier of the router's logits.",
        "random_logits": "Route at random (an ablation of learned routing).",
        "normalize_top_k": "Renormalise the picked weights to sum to one.",
        "routed_scaling_factor": "Multiplier of the routed experts' output.",
        "num_groups": "Experts are grouped; picks come from the best groups only.",
        "top_k_groups": "Groups a token may pick from.",
        "load_balancing": "`aux_loss` (a balancing loss), `aux_free` (a router bias stepped toward balance after each update) or `smebu` (the bias update with momentum and a soft clamp).",
        "bias_update_rate": "Step of the balancing bias.", "center_bias": "Keep the balancing bias at zero mean.",
        "bias_softclamp": "Soft clamp on the balancing bias.", "bias_momentum": "Momentum of the bias update.",
        "aux_loss_coef": "Weight of the load-balancing loss.",
        "aux_loss_scope": "Whether the loss balances the loads of the whole `batch` or of each `sequence`.",
        "latent_size": "LatentMoE: experts work in a smaller latent of this width.",
        "latent_input_norm": "Norm on the latent going into the experts.", "latent_output_norm": "Norm on the experts' latent output.",
        "expert_norm": "A norm inside every expert.", "shared_expert_sink": "The shared expert takes part in the router's softmax.",
        "num_zero_experts": "Experts that output zero: a pick of one skips compute for that slot.",
        "ffn_experts_per_token": "Target number of non-zero experts per token.",
    },
    "embed": {"max_positions": "Adds learned absolute positions up to this length.",
              "scale_by_sqrt_dim": "Multiply the embeddings by `sqrt(d_model)`.", "norm": "A norm on the embeddings.",
              "dropout": "Dropout on the embeddings."},
    "head": {"tied": "Use the embedding table transposed instead of a matrix of its own.", "bias": "A bias per token.",
             "softcap": "Soft cap on the logits.", "pointer": "Mix in a copy distribution over the context."},
    "linear": {"features": "Output channels.", "bias": "Add a bias."},
    "conv": {"size": "Taps.", "bias": "Add a bias."}, "short_conv": {"conv_size": "Taps.", "bias": "Add a bias."},
    "scale": {"init": "Initial value.", "per_channel": "One weight per channel."},
    "dropout": {"rate": "Probability of zeroing an element."},
    "value_embed": {"features": "Width of the embedding; `none` matches the values it is added to.", "std": "Initial standard deviation."},
    "rope": {"base": "The slowest frequency's period base.", "fraction": "Share of each head's channels that are rotated.",
             "layout": "`half` pairs channel i with i + d/2; `interleaved` pairs neighbours.",
             "scaling": "Frequency scaling for longer contexts: `pi`, `llama3` or `yarn`."},
    "indexer": {"num_heads": "Heads of the scorer.", "head_dim": "Channels per scorer head.", "top_k": "Keys (or blocks) kept per query.",
                "block_size": "Score blocks of this many keys instead of single keys.", "pool": "How a block's keys become its score: `mean` or `max`.",
                "per_group": "One pick per key/value group instead of one for all heads.", "relu": "ReLU on the per-head scores before they are summed.",
                "weighted": "Learned per-head weights from the query.", "norm": "Norm on the scorer's keys.",
                "loss_weight": "Weight of the loss that teaches the scorer the attention's own distribution.",
                "loss_over": "Whether that loss compares over the layer's `own` picks or the picks it was `served` through a port.",
                "candidate_block_size": "First stage of a two-stage pick: block size of the candidates.",
                "candidate_top_k": "Candidate blocks kept by the first stage."},
    "hc": {"expansion": "Copies of the stream.", "dynamic": "Weights depend on the input, not only on learned constants.",
           "sinkhorn_iters": "Sinkhorn iterations that make the mixing matrix doubly stochastic (`mhc`).",
           "single_pass": "Compute a block's read, write and mix weights in one projection."},
    "init": {"embed": "Applies to embedding tables.", "head": "Applies to heads.", "out": "Applies to projections that write the stream."},
    "fan": {"scale": "Variance multiplier.", "distribution": "`truncated` normal, `gaussian` or `uniform`."},
    "normal": {"std": "Standard deviation.", "truncate": "Truncate at this many standard deviations."},
    # ---- training
    "adamw": {"lr": "Peak learning rate; the schedule multiplies it.", "b1": "Decay of the first moment.", "b2": "Decay of the second moment.",
              "eps": "Added to the root of the second moment.", "weight_decay": "Decoupled decay, applied to matrices.",
              "cautious_weight_decay": "Decay only where the update and the weight agree in sign."},
    "muon": {"lr": "Peak learning rate of the orthogonalised updates.", "momentum": "Momentum of the gradient average.",
             "nesterov": "Use the Nesterov form of the momentum.", "ns_steps": "Newton-Schulz iterations.",
             "ns_coefficients": "The iteration's polynomial coefficients.", "ns_algorithm": "Which iteration: the quintic, or a variant.",
             "ns_restarts": "Restarts of the iteration.", "ns_dtype": "Dtype the iteration runs in.",
             "weight_decay": "Decoupled decay.", "cautious_weight_decay": "Decay only where update and weight agree in sign.",
             "consistent_rms": "Scale updates so their RMS matches AdamW's.", "adam": "The AdamW used for embeddings, heads, norms and scalars."},
    "normuon": {"b2": "Decay of the per-row second moment.", "eps": "Added to its root."},
    "ema": {"window": "The tail of the run the average covers: a number of steps, or a share of the run.", "blend": "The run ends on `last + blend * (average - last)`."},
    "schedule": {"warmup": "Steps of linear warm-up from zero.", "final": "The rate at the end, as a share of the peak.",
                 "shape": "The cool-down's curve."},
    "wsd": {"decay": "Share of the steps (or a number of steps) spent cooling down."},
    "cosine": {"horizon": "Steps the cosine is stretched over when they differ from the run's."},
    "documents": {"path": "A file or glob.", "column": "The column that holds the documents.",
                  "split": "The share of the documents (by content hash) this source reads: `(0, 0.99)`."},
    "text": {"bos": "Start every document with the tokenizer's bos token.", "eos": "End every document with its eos token."},
    "chat": {"template": "A built-in template's name or a Jinja template.", "train_on": "`assistant` replies, the `last` reply, or `all` tokens."},
    "tokens": {"path": "Files of raw ids.", "dtype": "The ids' integer type.", "header": "Bytes to skip at the start of each file."},
    "tokenizer": {"name": "A Hugging Face tokenizer folder or file, or `bytes`.", "bos": "The start token's text.", "eos": "The end token's text.",
                  "added": "Extra special tokens."},
    "packing": {"doc_mask": "Documents of a row attend only within themselves.", "chunk": "Tokens per shuffle chunk: the unit of packing and of a part file.",
                "long": "What becomes of a document longer than a row: `split`, `truncate` or `drop`.", "max_docs": "Most documents in one row.",
                "sort": "Place the longest documents first."},
    "checkpoint": {"every": "Steps between checkpoints.", "keep": "How many of the latest are kept."},
    "log": {"every": "Steps between log lines.", "trackers": "Where metrics also go: `wandb(...)`, `tensorboard`."},
    "eval": {"name": "Prefix of the metrics.", "data": "The held-out source.", "every": "Steps between evaluations.", "batches": "Batches per evaluation.",
             "seq_len": "Sequence length when it differs from training's.", "batch": "Batch size when it differs.", "positions": "Also report the loss of the targets at these positions."},
    "observe": {"every": "Steps between observations.", "histograms": "Also record histograms."},
    "profile": {"start": "First profiled step.", "steps": "Steps captured.", "tool": "The profiler: the framework's own trace, `nsys` or `ncu`.", "options": "Extra options for the tool."},
    "loss": {"z": "Weight of the z-loss (squared log-partition).", "mtp": "Weight of the multi-token-prediction heads' losses.", "prefix": "Adds prefix-token prediction (`prefix(...)`)."},
    "prefix": {"weight": "Weight of the prefix tokens' cross-entropy while it holds.", "hold": "Share of the run's steps the weight is held.", "decay": "Share of the steps after those over which it falls linearly to zero."},
    "phase": {"at": "First step of the phase (a step or a share of the run).", "seq_len": "New sequence length.", "batch": "New batch size.",
              "data": "New data.", "rope_scaling": "New RoPE scaling.", "rope_base": "New RoPE base."},
    "ramp": {"start": "Initial batch size.", "steps": "Steps to reach the full batch.", "multiple": "Batch sizes are multiples of this."},
    "precision": {"compute": "Dtype of activations and of matmuls that are not quantised.", "matmuls": "Format of the projections: `compute`, `mxfp8`, `nvfp4`.",
                  "roles": "Per-role overrides of `matmuls`.", "first": "Leading blocks kept in the compute dtype.", "last": "Trailing blocks kept in the compute dtype.",
                  "passes": "Which of fprop, dgrad and wgrad are quantised.", "switch": "A late change of `passes`.", "eval": "Format of evaluation forwards.",
                  "moments": "Dtype of the optimizer's moments.", "reduce": "Dtype gradients are reduced in.", "dispatch": "Format tokens travel to their experts in."},
    "switch": {"at": "Share of the run after which the new passes apply.", "passes": "The passes quantised from then on."},
    "mesh": {"data": "Replicas of the model (the batch is split).", "stage": "Pipeline stages.", "fsdp": "Ranks that shard parameters, gradients and moments.",
             "context": "Ranks that split each sequence.", "expert": "Ranks that split the experts.", "tensor": "Ranks that split heads and hidden units."},
    "methods": {"attention": "Which attention path runs.", "moe": "How tokens reach experts: `sorted` on one GPU; over the `expert` axis `fused_ep` (the in-kernel exchange over peer memory; `nccl_ep` names it too) or the library all-to-all (`all_to_all`, and every other name).",
                "capacity": "Rows an expert shard accepts, as a multiple of the even share.", "moe_chunks": "Token chunks the expert exchange is pipelined in.",
                "moe_stream": "Run the exchange on a side stream.", "remat": "`none`, `full` per block, `auto` (fitted to the memory), or a `remat(save=...)` policy.",
                "pipeline": "Pipeline schedule: `gpipe`, `1f1b`, `zbh1`, `circular`.", "stages": "Blocks per stage when the balance is set by hand.",
                "microbatches": "Microbatches a step's batch is split into.", "interleave": "Run each microbatch's forward beside the backward of the one before.",
                "tensor": "`gspmd` (library collectives) or `fused` (collectives inside the GEMM kernels).",
                "accumulate": "Whether microbatch gradients are summed `reduced` (sharded) or `unreduced` (whole, reduced once).",
                "loss": "Chunking of the head and the loss.", "orthogonalize": "How Muon's matrices are gathered for Newton-Schulz."},
    "remat": {"save": "Named activations kept for the backward.", "offload": "Named activations kept in host memory.", "first": "Blocks (from the first) the policy applies to."},
    "search": {"method": "The sampler.", "trials": "Trials in all.", "parallel": "Trials at once.", "halving": "Early stopping of trials.", "seed": "Seed of the sampler."},
    "halving": {"eta": "Share of trials kept at each rung is `1 / eta`.", "rungs": "Steps at which trials are compared.", "brackets": "Hyperband brackets."},
}

_AXES = "A mesh axis, a list of axes, or `none` for replicated."
FIELDS.update({
    "act": {"fn": "The function's name."},
    "dyt": {"alpha_init": "Initial `alpha`."},
    "nextn": {"norm": "The norm applied to the stream and to the next token's embedding before they are joined."},
    "engram": {"head_dim": "Channels per memory head.", "table_size": "Rows of each hash table.", "max_ngram_size": "Longest n-gram hashed.",
               "num_heads": "Hash functions (heads) per n-gram size.", "norm": "Norm on the stream before it gates the memory.",
               "conv_size": "Taps of the short convolution over the memory's output.", "vocab_classes": "Hash token classes instead of ids: the ids are folded to this many classes.",
               "boundary_token": "N-grams do not cross this token."},
    "doc_copy": {"gain": "Initial weight of the copy logits.", "lengths": "Context lengths whose matches are scored.", "counts": "Most matches counted per length."},
    "copy_pointer": {"dim": "Width of the pointer's queries and keys.", "token": "Copy only after this token.", "window": "Positions back the pointer can reach."},
    "attnres": {"block_size": "Blocks whose outputs are pooled into one history entry.", "norm_eps": "Epsilon of the history's norm."},
    "msar": {"block_size": "Blocks per history entry.", "kernel_sizes": "Pooling sizes of the history's scales.", "norm_eps": "Epsilon of the history's norm."},
    "gr": {"rank": "Rank of the gate's projection.", "expansion": "Copies of the stream.", "norm_eps": "Epsilon of the gate's norm."},
    "hc": {**FIELDS["hc"], "pre_bias": "Learned bias of the read weights.", "post_bias": "Learned bias of the write weights.",
           "res_bias": "Learned bias of the stream-mixing weights.", "norm_eps": "Epsilon of the norm in front of the dynamic weights."},
    "vpgate": {"temperature": "Temperature of the gate's sigmoid.", "eps": "Floor inside the variance-preserving normaliser."},
    "relbias": {"rank": "Rank of the bias as a function of the distance.", "extent": "Largest distance with a bias of its own."},
    "pi": {"factor": "Positions are divided by this."},
    "llama3": {"factor": "How much the low frequencies are slowed.", "original_max_len": "Context length the model was trained at.",
               "low_freq_factor": "Wavelengths longer than `original_max_len / low_freq_factor` are scaled fully.",
               "high_freq_factor": "Wavelengths shorter than `original_max_len / high_freq_factor` are kept."},
    "yarn": {"factor": "Context extension factor.", "original_max_len": "Context length the model was trained at.",
             "beta_fast": "Rotations above which a frequency is kept.", "beta_slow": "Rotations below which it is interpolated.",
             "attention_factor": "Attention temperature; `none` derives it from `factor`.",
             "attention_factor_on": "Apply the temperature to the `rotary` embeddings or to the `softmax` scale."},
    "indexer": {**FIELDS["indexer"], "rope_layout": "Pairing of the rotated channels in the scorer."},
    "power": {"a": "Scale of the power law.", "b": "Its exponent.", "decay": "Share of the steps spent cooling down."},
    "multistep": {"at": "Shares of the run at which the rate drops.", "factor": "Multiplier at each drop."},
    "piecewise": {"pieces": "The pieces, in order."},
    "piece": {"until": "Share of the run the piece ends at.", "to": "Rate (as a share of the peak) reached at its end; `none` keeps the current one.",
              "shape": "Curve from the current rate to `to`."},
    "layout": {k: v + " " + _AXES for k, v in {
        "batch": "Shards the rows of a batch.", "seq": "Shards the tokens of a row.", "stream": "Shards the residual stream between layers (sequence parallelism).",
        "embed": "Shards the channel axis of weights.", "vocab": "Shards the vocabulary axis of embedding and head.", "heads": "Shards attention heads.",
        "kv_heads": "Shards key/value heads.", "mlp": "Shards feed-forward hidden units.", "experts": "Shards the experts.", "latent": "Shards latent projections.",
        "layers": "Shards the stacked layers axis.", "stages": "Assigns blocks to pipeline stages.",
        "fsdp": "Shards parameters, gradients and optimizer state."}.items()} | {"zero": "`3` shards parameters too; `1` shards only the optimizer state."},
    "roles": {k: f"Format of the {v} projections; `none` follows `precision.matmuls`." for k, v in {
        "q": "query", "kv": "key and value", "o": "attention output", "mlp": "feed-forward", "experts": "routed experts'", "latent": "low-rank latent",
        "recurrence": "recurrent mixers' input", "recurrence_out": "recurrent mixers' output", "mtp": "multi-token-prediction"}.items()},
    "methods": {**FIELDS["methods"], "recurrence": "How linear recurrences are evaluated: a chunked `scan` or a fused kernel.",
                "states": "`keep` the chunk states for the backward or `recompute` them.", "repeat": "Run a repeat `unroll`ed or as a loop over stacked weights.",
                "rounds": "Rounds of a circular pipeline.", "tensor_chunks": "Chunks the tensor-parallel collectives are pipelined in.",
                "gather": "Gather sharded parameters once a `step` or `layer` by layer.", "donate": "Update the state in place."},
    "compiler": {"preset": "A named set of build options.", "options": "Free-form flags, e.g. `--fsdp=fused`.",
                 "reductions": "`early`: reduce gradients while the backward runs."},
    "uniform": {"low": "Lower end.", "high": "Upper end."}, "log_uniform": {"low": "Lower end (positive).", "high": "Upper end."},
    "int_uniform": {"low": "Lower end.", "high": "Upper end (inclusive).", "log": "Sample uniformly in the logarithm."},
    "choice": {"options": "The values to choose from."},
    "gp": {"startup": "Random trials before the model is used.", "acquisition": "`log_ei` (expected improvement) or `ucb`.", "beta": "Exploration weight of `ucb`."},
    "tpe": {"startup": "Random trials before the estimator is used.", "candidates": "Candidates drawn per suggestion.", "gamma": "Share of trials counted as good.",
            "multivariate": "Model the dimensions jointly."},
    "wandb": {"project": "Project name.", "entity": "Team or user.", "group": "Group of the run.", "tags": "Tags of the run.", "mode": "`online`, `offline` or `disabled`."},
})

# ---- notes checked field by field against what the layers compute
FIELDS["attention"].update({
    "output_norm": "A norm of each head's output, before the gate.",
    "gated": "An elementwise gate `act(W x)` from the layer's input on each head's output, before the output projection.",
    "gate_input_rank": "The gate's projection of the input made low-rank (`silu(x W_d) W_u`, `W_d` of this many columns per head).",
    "gate_output_rank": "The gate also reads the head's own output through a low-rank map of this rank, added to its logits before the activation.",
    "gate_cross_head": "A second gate, one value per head, from all the heads' outputs together; it multiplies the first.",
    "log_scale": "Logits times `1 + log_scale * ln(max(n / log_scale_floor, 1))` at the query's position `n` (from 1), so attention stays sharp at long range.",
    "log_scale_floor": "Positions up to this one keep their logits' scale.",
})
FIELDS["gqa"].update({
    "bias": "Biases on the projections of the input: q, k, v and the gate.",
    "output_bias": "A bias on the output projection; `none` follows `bias`.",
    "power_scale": "Queries times `(1 + n / power_scale_length) ** power_scale` at their position `n` (from 1): keeps attention without RoPE sharp at long range.",
    "power_scale_length": "The position at which the queries' scale reaches `2 ** power_scale`.",
    "kv_conv_size": "A causal depthwise convolution of this many taps on keys and values, added to them: `k + conv(k)`.",
    "exclusive": "Exclusive self-attention: each head's output less its part along the query's own value, `y - (y . v) v / (v . v)`, before the output's norm and gate; `learned` scales what is taken off by a learned factor.",
    "k_eq_v": "Values come from the key projection (no v projection): each head's projected key, normalised without a gain and not rotated.",
    "differential": "Differential attention: twice the query heads, each output `a1 - sigmoid(x W) a2` of a pair of heads.",
    "paired": "Paired-head attention: two query heads (and two key/value heads) are interleaved along the sequence into one of twice the length, so a query sees both heads' keys.",
    "mimetic_vo": "Mimetic initialisation of V and O at this beta: their kernels start as blocks of `+sqrt(beta)` and `-sqrt(beta)` identities.",
    "mimetic_noise": "Standard deviation of the noise on V and O under `mimetic_vo`.",
    "qk_norm_all_heads": "`qk_norm` over all the heads' channels together (one norm of the queries, one of the keys), before they split into heads.",
})
FIELDS["mla"].update({"rope": "On the decoupled `qk_rope_head_dim` part; `none` rotates nothing.",
                      "q_lora_rank": "Width of the latent the queries come from; `none` for a full-rank query projection."})
FIELDS["csa"].update({
    "head_dim": "Width of a query head and of a latent (the heads share the latents as their one key/value head).",
    "compress_ratio": "Tokens pooled into one compressed latent; `none` keeps the window only.",
    "latent_norm": "Norm of the query latent, the latents, the compressed ones and the indexer's keys.",
    "o_lora_rank": "Grouped low-rank output projection: `o_groups` groups of heads, each projected to this rank, then mixed back to the width; `none` for one dense projection.",
})
FIELDS["mlp"].update({
    "dropout": "Dropout rate of the output, in training.",
    "limit": "Clamped GLU: the gate's input is capped at `limit`, the up branch at `+-limit`.",
    "up_softcap": "Soft cap of the up branch, `cap * tanh(up / cap)`.",
    "up_offset": "Added to a gated MLP's up branch after it is clipped (gpt-oss: `up + 1`).",
})
FIELDS["moe"].update({
    "num_shared_experts": "Experts every token goes through, run as one MLP of that many times the shared expert's hidden width.",
    "router": "How logits become scores: a `softmax` over the experts, a `sigmoid` each, or `sqrt(softplus(.))` each.",
    "router_bias": "A learned bias on the router's logits (unlike `aux_free`'s, which only steers the choice).",
    "routed_scaling_factor": "Multiplies the picked weights.",
    "random_logits": "For benchmarks: a training forward routes by random logits, so every expert takes an even share of the picks and a capacity drops few.",
    "num_groups": "Group-limited routing: the experts are in this many groups, each scored by the sum of its two best experts.",
    "top_k_groups": "Groups each token picks its experts from.",
    "load_balancing": "`aux_loss`: a balance loss. `aux_free`: a bias per expert on the scores that pick the top-k (not on the weights), moved after every step toward even loads. `smebu`: that move with momentum and a tanh soft clamp.",
    "bias_update_rate": "How far the balancing bias moves per training step (`smebu`: at most).",
    "center_bias": "`aux_free`: subtract the bias's mean after every move (`smebu` always does).",
    "bias_softclamp": "`smebu`'s kappa: how soon the tanh of the load's deviation saturates.",
    "bias_momentum": "`smebu`'s beta: the decay of the running average of the moves.",
    "aux_loss_coef": "Weight of each layer's balance loss `E * sum_e f_e P_e` (share of picks times mean score per expert).",
    "latent_size": "LatentMoE: routed experts run in a narrower space of this width between a down and an up projection; the router and shared experts see the full width.",
    "latent_input_norm": "LatentMoE: a norm of the tokens after the down projection.",
    "latent_output_norm": "A norm of the routed sum, before LatentMoE's up projection.",
    "expert_norm": "A norm of each routed expert's output.",
    "shared_expert_sink": "The shared experts are weighted by the router too, normalised with the top-k; otherwise they are added with weight 1.",
    "num_zero_experts": "Zero-computation experts: identity experts the router scores after the routed ones; a pick of one passes the token through as it is, times its weight, and runs no FFN.",
    "ffn_experts_per_token": "The FFN experts a token goes through on average, which the balancing steers toward; `none` is what uniform picks give.",
})
FIELDS["recurrent"].update({
    "head_dim": "Width of a query and a key head: the state's rows.",
    "v_head_dim": "Width of a value head: the state's columns; `none` is `head_dim`.",
    "num_v_heads": "Value heads; with more of them than query/key heads, each query/key head serves a group of them.",
    "conv_size": "Taps of a causal depthwise convolution on q, k and v (each then SiLU'd); `none` for none.",
    "output_gate": "Activation of a gate on the output, after its norm and before the output projection; `none` for no gate.",
    "gate_rank": "Rank of the decay's projection.",
    "output_gate_rank": "Rank of the output gate's projection; `none` for full rank.",
    "gate_lower_bound": "Bounded decay `lower_bound * sigmoid(.)` in `(lower_bound, 0)` instead of `-exp(A) * softplus(.)`; `none`: unbounded.",
    "negative_eigenvalues": "The erase gate times 2, in (0, 2), so the state's transition may have negative eigenvalues.",
})
FIELDS["rwkv7"].update({"gate_rank": "Rank of the output gate's projection.", "output_gate": "The output gate is `act(x G1) G2` with this activation between.",
                        "conv_size": "`none` only: RWKV-7 shifts tokens instead of convolving.",
                        "norm_eps": "Epsilon of each head's output layer norm, times the value head's width.", "v_rank": "Rank of the value residual's mix (with the `v` port)."})
FIELDS["mamba2"].update({"state_size": "State dims of each inner channel (the papers' N).", "num_heads": "`none` is `expand * width // head_dim`.",
                         "num_groups": "Groups that share B and C, as key/value heads are shared in GQA."})
FIELDS["mamba"].update({"state_size": "State dims of each inner channel (the papers' N).", "dt_min": "The time steps start log-uniform in `[dt_min, dt_max]`.",
                        "dt_max": "The largest time step at the start."})
FIELDS["conv"].update({"size": "Taps: each position sees itself and the `size - 1` before it."})
FIELDS["short_conv"].update({"bias": "Biases on the projections and the convolution."})

FIELDS["engram"].update({"norm": "Norm of the stream (the query), of the keys, and of the memory's output before the convolution.",
                         "conv_size": "Taps of the causal convolution over the memory's output, zero-initialised and dilated by `max_ngram_size`; `none` for none.",
                         "vocab_classes": "Hash each token's class (of this many) instead of its id: id `i` is class `i mod vocab_classes`; `none`: the ids.",
                         "boundary_token": "N-grams do not reach back past this token (an end-of-text token, say); `none`: no boundary.",
                         "table_size": "Rows of each head's table: the least prime at or above this that no earlier head has taken.",
                         "head_dim": "Width of a table row.", "num_heads": "Hash heads per n-gram size, each with a table of its own."})
FIELDS["doc_copy"].update({"gain": "The copy vector's weight at this site, learned from here.", "lengths": "The context lengths that can match, shortest first.",
                           "counts": "How many earlier occurrences of a matched context the buckets tell apart (1, 2 and 3 or more by default)."})
FIELDS["copy_pointer"].update({"token": "The vocabulary row of the `<copy>` token, one that no real token is; `none`: the last row.",
                               "window": "How far back the pointer looks, in tokens; `none`: the whole document."})
FIELDS["rope"].update({"base": "Theta, the base of the frequencies (Llama 3: 500000).",
                       "fraction": "Partial rotary: only this share of each head's dims is rotated, the first ones, in whole pairs."})
FIELDS["pi"].update({"factor": "How many times longer the context gets: frequencies are divided by it."})
FIELDS["yarn"].update({"factor": "How many times longer than `original_max_len` the context gets.",
                       "beta_fast": "Pairs that turn more times than this over the original length keep their frequency.",
                       "beta_slow": "Pairs that turn fewer times than this have their frequency divided by `factor`.",
                       "attention_factor": "YaRN's temperature (q . k is scaled by its square); `none` is `0.1 * ln(factor) + 1`; 1 disables it.",
                       "attention_factor_on": "`rotary` multiplies cos and sin by it (the rotated dims only); `softmax` multiplies the softmax scale by its square (all dims)."})
FIELDS["llama3"].update({"factor": "What the slowest pairs' frequencies are divided by.",
                         "low_freq_factor": "Pairs that turn fewer times than this over the original length are divided by `factor`.",
                         "high_freq_factor": "Pairs that turn more times than this keep their frequency; between the two the scaling is blended."})
FIELDS["relbias"].update({"rank": "Width of the table's entries and of each head's projection.", "extent": "Offsets (from 0) that have a bias; farther keys get none."})
FIELDS["indexer"].update({
    "top_k": "Keys each query keeps (in whole blocks, with `block_size`).",
    "block_size": "Pick whole blocks of this many keys (`top_k` keys in total), scored as `pool` says.",
    "pool": "How a block scores: `mean` pools its keys into one, which a query scores once the block is complete (its own unfinished block is kept beside the picks); `max` is its best key's score.",
    "per_group": "A pick for each key/value head's group of query heads, by an indexer head of its own; else one pick for all heads.",
    "relu": "ReLU on each head's dot products; else the plain ones.", "weighted": "Learned per-head score weights; else a plain sum.",
    "norm": "Norm of each query head and of the keys (after block pooling); `none`: no query norm and the layer's own key norm.",
    "rope_layout": "How the indexer pairs RoPE dims when its keys are the tokens, whatever the layer's own layout.",
    "candidate_block_size": "What a `candidates` port exports: the best `candidate_top_k` blocks of this many keys, each scored by its best key.",
    "candidate_top_k": "Blocks in the candidate pool.",
    "loss_weight": "Weight of the indexer's loss, its only training signal: the KL divergence from the attention over the kept keys to the softmax of its scores. 0 leaves it untrained.",
    "loss_over": "Whose attention the loss distils: `own`, its layer's; `served`, also that of every layer that reads its picks through the `index` port.",
})
FIELDS["hc"].update({
    "expansion": "Copies of the stream, 2 or more: one is the plain residual stream.",
    "dynamic": "Coefficients that depend on the stream (a projection that starts at 0) on top of static ones; else static ones alone.",
    "pre_bias": "`mhc`: the static read logits start at this on the k-th branch's own stream and at minus it on the others.",
    "post_bias": "As `pre_bias`, for `mhc`'s static write logits.",
    "res_bias": "`mhc`: the static mixing logits off the diagonal (0 on it): the mixing starts as the identity to within `e^res_bias`.",
    "single_pass": "A branch reads with the coefficients the branch before it computed.",
    "norm_eps": "Epsilon of the norm before the dynamic coefficients."})
FIELDS["gr"].update({"rank": "Rank of the read gate.", "norm_eps": "Epsilon of the streams' RMS norm."})
FIELDS["attnres"].update({"block_size": "Branch outputs summed into one source; `none`: each is its own source.", "norm_eps": "Epsilon of the keys' RMS norm."})
FIELDS["msar"].update({"block_size": "Branch outputs summed into one source; `none`: each is its own source.",
                       "kernel_sizes": "Taps of each stream's convolution after the first (which is the source as it is): 4, 8 and 12 make four streams.",
                       "norm_eps": "Epsilon of the keys' and the mixer's RMS norms."})
FIELDS["vpgate"].update({"temperature": "Divides the learned `g` inside the gate's sigmoid.", "eps": "`a = sqrt(max(1 - b^2, eps))`: the stream is never cut off."})
FIELDS["init"].update({"embed": "How the embedding tables start (the tokens' and the learned positions'; a tied head reads the tokens'); `none`: as the rest.",
                       "head": "How an untied head starts; `none`: as the rest.",
                       "out": "How the projections back to the stream's width start (attention's and the mixers' outputs, MLPs' and experts' down); `none`: as the rest."})
FIELDS["fan"].update({"scale": "The variance times the fan.", "distribution": "What it draws from at that variance: a normal `truncated` at 2 standard deviations, a `gaussian`, or a `uniform`."})
FIELDS["normal"].update({"std": "The standard deviation, before truncation.", "truncate": "Values farther than this many standard deviations from 0 are drawn again; `none`: none are."})

FIELDS["documents"].update({"path": "A glob of parquet (or JSON-lines) files, relative to the working directory.",
                            "split": "The documents whose content hash falls in `[start, end)`: `(0.99, 1)` is a 1% held out."})
FIELDS["text"].update({"column": "The column that holds each document's text."})
FIELDS["chat"].update({"column": "The column that holds each conversation's messages.",
                       "train_on": "`assistant`: every reply; `last`: the last reply alone; `all`: every token, prompts and template too."})
FIELDS["tokens"].update({"path": "A glob of shards of raw token ids.", "header": "Bytes before the tokens in every shard."})
FIELDS["tokenizer"].update({"bos": "The token a document starts with, where its source sets `bos`.", "eos": "The token a document ends with, where its source sets `eos`.",
                            "added": "Special tokens appended after the vocabulary, for a chat template the tokenizer lacks."})
FIELDS["packing"].update({"doc_mask": "Positions restart at every document and attention stays within it.", "chunk": "About how many tokens of documents are packed together (and make one part file).",
                          "long": "A document longer than a row: `drop`ped, `truncate`d to a row, or `split` into pieces that fill rows.",
                          "max_docs": "The most documents (and pieces of them) in a row; `none`: as many as fit.", "sort": "Longest first; `false` keeps the shuffled order (online best fit)."})
FIELDS["adamw"].update({"weight_decay": "Decoupled decay of the matrices, times the learning rate.",
                        "cautious_weight_decay": "Decay only the entries whose update has the parameter's sign (or is 0), so decay never pulls against the step."})
FIELDS["muon"].update({
    "momentum": "Decay of the gradients' average that is orthogonalised.", "nesterov": "Nesterov's look-ahead.",
    "ns_coefficients": "The iteration's quintics by name: one set for every iteration (`jordan`), or one per iteration (`polar_express`).",
    "ns_algorithm": "How it iterates: `standard`, or `gram` on the Gram matrix of each matrix's shorter side (fewer products the less square a matrix is).",
    "ns_restarts": "The iterations after which `gram` restarts from the matrix so far; `none`: after the second and every third after it.",
    "ns_dtype": "What Newton-Schulz runs in, and what the updates move between devices in.",
    "consistent_rms": "Updates scaled to this RMS, as AdamW's roughly are, so one learning rate suits both; `none`: scaled by `sqrt(max(1, fan_out / fan_in))`.",
    "adam": "The AdamW of everything Muon does not take (embeddings, heads, norms, scalars); `none`: `adamw(lr=lr)`."})
FIELDS["normuon"].update({"b2": "Decay of each neuron's mean-square average.", "eps": "Added to that average's root."})
FIELDS["ema"].update({"window": "The steps it averages, the run's last (a number, or a share of the steps below 1); a step's weights join at the rate `2 / (window + 1)`.",
                      "blend": "How much of the average the run ends on: `last + blend * (average - last)`; 1 ends on the average alone."})
FIELDS["schedule"].update({"warmup": "Steps of linear warm-up, or a share of the steps below 1.", "final": "The multiplier at the last step: a fraction of the peak."})
FIELDS["wsd"].update({"decay": "The share of the steps the cool-down takes."})
FIELDS["cosine"].update({"horizon": "The share of the steps at which the cosine reaches `final`: above 1 the run stops before it does, below 1 it holds there."})
FIELDS["power"].update({"a": "The power law's amplitude, for a batch of one row.", "b": "Its exponent, of the tokens trained.", "decay": "The share of the steps the cool-down takes."})
FIELDS["multistep"].update({"at": "The shares of the steps at which the rate drops, in order.", "factor": "What each drop multiplies the rate by."})
FIELDS["piecewise"].update({"pieces": "The pieces in order, each ending later than the one before; the last at 1."})
FIELDS["piece"].update({"to": "The multiplier it ends at; `none` holds where it starts.", "shape": "How it gets there; `constant` is there at once."})
FIELDS["phase"].update({"at": "The step it starts at, or a share of the steps (0.9 starts the last tenth).", "seq_len": "Tokens per row; `none`: as before.",
                        "batch": "Rows per step; `none`: as before.", "data": "A source or a mixture; `none`: as before.",
                        "rope_scaling": "The RoPE scaling of full-attention layers from then on.", "rope_base": "The RoPE base of full-attention layers from then on (raised for long context)."})
FIELDS["ramp"].update({"start": "Rows per step at the first step.", "steps": "The steps it takes to reach the run's batch.", "multiple": "The batch sizes it takes are multiples of this; `none`: of `start`."})
FIELDS["loss"].update({"z": "Weight of the z-loss, `log(Z)^2` of the first head.", "mtp": "Weight of the mean loss of the heads that predict further ahead.",
                       "prefix": "The first head also predicts each target's prefix token, as `prefix(...)` says; `none`: not."})
FIELDS["eval"].update({"name": "What its metrics' names start with (`eval_loss`, `eval_bpb`).", "data": "A source or a mixture, as `data` takes.",
                       "batches": "Batches an evaluation reads, the same ones each time.",
                       "positions": "Where buckets of targets by position in their document start, after the first at 0: `[2048, 8192]` also logs `..._0`, `..._2k`, `..._8k`."})
FIELDS["wandb"].update({"group": "`none`: the file's name, which a sweep's runs share.", "entity": "The team or user it is under; `none`: your default.",
                        "mode": "`online`: as it trains; `offline`: into the run's directory, to sync later; `disabled`: nowhere; `none`: as `WANDB_MODE` says."})
FIELDS["observe"].update({"every": "Steps between the steps that observe the model.", "histograms": "Take histograms of the stream and the gradients too."})
FIELDS["profile"].update({"start": "The step after which the trace starts.", "steps": "The steps it traces.", "options": "More flags for nsys or ncu, as its command line writes them."})
FIELDS["precision"].update({
    "compute": "The dtype the forward and backward passes run in.",
    "matmuls": "The format the projections inside blocks multiply in: `compute`, `mxfp8`, `mxfp8_2d` or `nvfp4`.",
    "roles": "A format by the kind of projection (`roles(...)`).",
    "first": "The residual branches outside any other at the start of the model that multiply in `compute`: a number of them, or a share (rounded up).",
    "last": "As `first`, the last ones before the first head.", "passes": "The GEMMs (fprop, dgrad, wgrad) that multiply in the format.",
    "eval": "Evaluation multiplies as training does, or in `compute`.",
    "moments": "The dtype the optimizer's moments are kept in between steps (they update in float32).",
    "reduce": "The dtype gradients are summed over the ranks in: `compute`, or `float32`.",
    "dispatch": "What the expert exchange sends tokens to their experts in: `compute`, or MXFP8; what comes back, and gradients, go in `compute`."})
FIELDS["roles"].update({"q": "Attention's queries and gate (gqa, mla, csa, the indexer); `none` follows `precision.matmuls`.", "kv": "Attention's keys and values.",
                        "o": "Attention's output projection.", "mlp": "MLPs, the shared experts' too.",
                        "experts": "The routed experts' grouped GEMMs: `compute`, `mxfp8` or `mxfp8_2d`; `none` is `matmuls` where it is one of those, else `compute`.",
                        "latent": "LatentMoE's projections to and from its latent.", "recurrence": "The recurrent mixers' projections, but the output.",
                        "recurrence_out": "The recurrent mixers' output projection.", "mtp": "`nextn`'s projection, and every branch after the first head."})
FIELDS["switch"].update({"passes": "The GEMMs in the format after it; `[]` is none."})
FIELDS["mesh"].update({"data": "Copies of the model; `none`: the devices that are left.", "fsdp": "Devices that split parameters (and rows of the batch).",
                       "context": "Devices a row's positions split over.", "expert": "Devices the routed experts split over (and rows of the batch).",
                       "tensor": "Devices heads, hidden units and the vocabulary split over."})
FIELDS["layout"].update({"seq": "Positions, inside a layer. " + _AXES, "stream": "Positions of the residual stream, between branches (sequence parallelism). " + _AXES,
                         "embed": "The model's width. " + _AXES, "latent": "Low-rank bottlenecks (MLA, LatentMoE). " + _AXES,
                         "layers": "The stacked passes of a repeat run as a loop. " + _AXES, "stages": "The passes of a pipelined repeat, a share per stage. " + _AXES,
                         "fsdp": "What sharding splits a parameter's first dimension over: the axes that copy dense parameters, but `data` (which HSDP keeps as copies)."})
FIELDS["remat"].update({"save": "Kept on the device for the backward: `attention`, `recurrence`, ...", "offload": "Moved to the host's memory until the backward reads them.",
                        "first": "The passes of each repeat it recomputes, from the first; the rest keep everything. `none`: every pass."})
FIELDS["methods"].update({
    "attention": "The attention path: `auto` (the kernels where they take the call); over `context`: `ulysses`, `gathered` or `ring`.",
    "capacity": "The picks an expert rank takes from each peer, as a multiple of its even share; what does not fit is dropped (the `dropped` metric).",
    "moe_chunks": "The slices of each rank's tokens that expert parallelism sends one after another, so one's exchange runs beside another's experts.",
    "recurrence": "The linear recurrences: `scan`, all of a row's positions on each rank; over `context`, each rank's positions continue from the state the ranks before pass on.",
    "states": "What a chunked recurrence's backward reads of its chunks' states: `keep`, from the forward, or `recompute`, from its inputs (less memory, more time).",
    "repeat": "A repeat's passes: `unroll`, a module each, run in a row.", "rounds": "Times a circular pipeline sends a microbatch round.",
    "stages": "The passes of the pipelined repeat each stage runs, first to last; `none`: the split that balances the stages.",
    "orthogonalize": "How Muon reaches whole matrices under sharding: `gather`, each whole on every rank that holds a part; `owner`, each whole on one rank.",
    "loss": "How the loss takes a head's logits: `chunks`, a chunk of positions at a time, never all of them; `logits`, whole.",
    "microbatches": "The microbatches a step takes its batch in, adding up their gradients; under a pipeline, those it sends through its stages.",
    "gather": "Where a step runs its layers more than once, sharded parameters are gathered once a `step`, or as each `layer` runs (one layer's held at a time).",
    "accumulate": "How microbatch gradients add up: `unreduced`, each rank's own, reduced once a step; `reduced`, every microbatch; `auto` chooses.",
    "donate": "A step's new state takes the old one's memory."})
FIELDS["compiler"].update({"reductions": "Where the step's gradient reductions start: `early`, each as its gradient is computed, or after the backward."})
FIELDS["choice"].update({"options": "The options' names, or the options as written: `swish`, `gelu`."})
FIELDS["tpe"].update({"startup": "Quasi-random trials before the densities propose.", "candidates": "Points drawn from the best trials' density, to pick from.",
                      "gamma": "The share of the trials that count as the best.", "multivariate": "One density over every dimension (it sees how they interact), or one each."})
FIELDS["gp"].update({"startup": "Quasi-random trials before the GP proposes.", "acquisition": "What the next point maximises: expected improvement in logs (`log_ei`), or the upper confidence bound (`ucb`).",
                     "beta": "`ucb`'s weight of the deviation: mean + beta * deviation."})

TRAIN_FIELDS = {
    "data": "What the model trains on: `text(...)`, `chat(...)`, `tokens(...)`, `synthetic`, or a weighted mixture.",
    "tokenizer": "The tokenizer of document sources.", "packing": "How documents become rows of `seq_len` tokens.",
    "optimizer": "`adamw(...)`, `muon(...)` or `normuon(...)`.", "schedule": "The learning-rate schedule (a multiplier of `optimizer.lr`).",
    "seq_len": "Tokens per row.", "batch": "Rows per step, over all GPUs.", "batch_ramp": "Grow the batch over the first steps.",
    "steps": "Optimizer steps.", "curriculum": "Phases that change data, length, batch or RoPE during the run.", "seed": "Seed of initialisation and data order.",
    "clip": "Clip the global gradient norm to this value.", "ema": "Keep a moving average of the weights.", "loss": "Extra loss terms.",
    "eval": "Periodic evaluations.", "checkpoint": "Periodic checkpoints.", "log": "Logging.", "observe": "Forward-pass statistics.", "profile": "A profiler capture.",
    "precision": "Dtypes and matmul formats.", "mesh": "GPUs per parallel axis.", "layout": "Which mesh axis shards what.", "methods": "Algorithm choices.",
    "compiler": "Build options.", "objective": "The metric a sweep or search ranks runs by.", "search": "A hyper-parameter search.",
}

MODEL_SETTINGS = {
    "d_model": "Width of the residual stream.", "vocab_size": "Size of the vocabulary.",
    "residual": "The residual algebra every `[branch]` uses: plain addition when unset, or `hc`, `mhc`, `gr`, `attnres`, `msar`, `vpgate`.",
    "init": "How weights are initialised, per role.", "model": "The graph that is built: layers composed left to right.",
}


def note(tag: str, field: str) -> str:
    """The catalogue's note on `tag.field`: the tag's own entry, else its families'."""
    own = FIELDS.get(tag, {}).get(field)
    if own:
        return own
    for family, tags in FAMILIES.items():
        if tag in tags and field in FIELDS.get(family, {}):
            return FIELDS[family][field]
    return ""
