"""Make the golden files of this folder: logits of the REFERENCE engine's own C code
(lawnak/FastGGUF, fastgguf.c ``forward``) on a tiny random Llama, to anchor the plain
implementation in ``tests/plain_llama.py``.

    python tests/golden/make_golden.py /path/to/FastGGUF

What it does
1. writes a tiny random model folder (``tiny_model/``: config.json + float32 model.safetensors)
   with sizes that are no powers of two, one KV head, llama3 rotary scaling, untied head;
2. exports it as a float32 GGUF file with the reference's tensor names (fastgguf.c:4266-4278,
   :4292-4365) and metadata keys (:4213-4229).  The reference rotates ADJACENT pairs for
   ``llama`` (fastgguf.c:4198, :3138-3139) while model folders pair (j, j + hd/2), so the rows of
   every head of Wq and Wk are permuted: new row 2j <- old row j, new row 2j+1 <- old row
   j + hd/2 (scores do not change under a common permutation of q and k).  The llama3 divisors
   go in as ``rope_freqs.weight`` (:4278, :3131);
3. compiles ``ref_harness.c`` against the reference source and runs it token by token;
4. stores ``tiny_ref_logits.f32`` ([T, vocab] float32) and ``tiny_tokens.json``.

Needs gcc and the ``gguf`` Python package; the committed outputs let the tests run without them.
"""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, ".."))

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 40, "num_hidden_layers": 2, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 16, "intermediate_size": 56, "vocab_size": 67, "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 16},
    "max_position_embeddings": 128, "tie_word_embeddings": False, "torch_dtype": "float32",
    "hidden_act": "silu",
}
TOKENS = [(i * 37 + 11) % 67 for i in range(24)]


def main():
    ref_dir = sys.argv[1]
    from fastgguf_b200.registry import config_from_dict
    from fastgguf_b200.weights import write_random_model
    import plain_llama
    from gguf import GGUFWriter

    model_dir = os.path.join(HERE, "tiny_model")
    write_random_model(config_from_dict(CONFIG), 3, model_dir, "float32")
    cfg, W = plain_llama.read_model_folder(model_dir)
    E, H, KV, hd = plain_llama.sizes(cfg)

    def permute(w, heads):           # halves layout -> adjacent pairs, per head
        w = w.reshape(heads, 2, hd // 2, w.shape[1])        # [head, half, j, in]
        return w.permute(0, 2, 1, 3).reshape(heads * hd, -1).contiguous()

    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "tiny.gguf")
        w = GGUFWriter(path, "llama")
        w.add_block_count(cfg["num_hidden_layers"]); w.add_context_length(cfg["max_position_embeddings"])
        w.add_embedding_length(E); w.add_feed_forward_length(cfg["intermediate_size"])
        w.add_head_count(H); w.add_head_count_kv(KV); w.add_key_length(hd); w.add_value_length(hd)
        w.add_layer_norm_rms_eps(cfg["rms_norm_eps"]); w.add_rope_freq_base(cfg["rope_theta"])
        w.add_rope_dimension_count(hd)
        f32 = lambda t: t.to(torch.float32).numpy()
        w.add_tensor("token_embd.weight", f32(W["model.embed_tokens.weight"]))
        w.add_tensor("output.weight", f32(W["lm_head.weight"]))
        w.add_tensor("output_norm.weight", f32(W["model.norm.weight"]))
        w.add_tensor("rope_freqs.weight", np.asarray(plain_llama.plain_rope_divisors(cfg, hd), dtype=np.float32))
        for i in range(cfg["num_hidden_layers"]):
            p, b = f"model.layers.{i}.", f"blk.{i}."
            w.add_tensor(b + "attn_norm.weight", f32(W[p + "input_layernorm.weight"]))
            w.add_tensor(b + "attn_q.weight", f32(permute(W[p + "self_attn.q_proj.weight"], H)))
            w.add_tensor(b + "attn_k.weight", f32(permute(W[p + "self_attn.k_proj.weight"], KV)))
            w.add_tensor(b + "attn_v.weight", f32(W[p + "self_attn.v_proj.weight"]))
            w.add_tensor(b + "attn_output.weight", f32(W[p + "self_attn.o_proj.weight"]))
            w.add_tensor(b + "ffn_norm.weight", f32(W[p + "post_attention_layernorm.weight"]))
            w.add_tensor(b + "ffn_gate.weight", f32(W[p + "mlp.gate_proj.weight"]))
            w.add_tensor(b + "ffn_up.weight", f32(W[p + "mlp.up_proj.weight"]))
            w.add_tensor(b + "ffn_down.weight", f32(W[p + "mlp.down_proj.weight"]))
        w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(progress=False); w.close()

        exe = os.path.join(tmp, "harness")
        subprocess.run(["gcc", "-O2", "-fopenmp", "-I", ref_dir, os.path.join(HERE, "ref_harness.c"), "-o", exe,
                        "-lm", "-ldl"], check=True)
        out = os.path.join(HERE, "tiny_ref_logits.f32")
        env = dict(os.environ, FASTGGUF_GPU="off", OMP_NUM_THREADS="1")
        subprocess.run([exe, path, out] + [str(t) for t in TOKENS], check=True, env=env,
                       stdout=subprocess.DEVNULL)
    with open(os.path.join(HERE, "tiny_tokens.json"), "w") as f:
        json.dump({"tokens": TOKENS, "vocab_size": cfg["vocab_size"]}, f)
    ref = np.fromfile(out, dtype="<f4").reshape(len(TOKENS), cfg["vocab_size"])
    mine = plain_llama.plain_forward(cfg, W, TOKENS, torch.float64).numpy()
    print("reference vs plain (float64): max |dlogit| = %.3e, max |logit| = %.3f"
          % (np.abs(ref - mine).max(), np.abs(ref).max()))


if __name__ == "__main__":
    main()
