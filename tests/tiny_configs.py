"""Small Qwen3 configurations for tests.  They differ from one another in every
size and option: layers, width, head counts and groups (GQA, MQA, 2:1), head
size (also one that is no power of two), heads * head size equal to the width or
not, intermediate size, vocabulary (also an odd one), rope theta, eps, position
limit, tied or untied output, no window or a window on some layers."""
import copy


def _base(**kw):
    d = {
        "architectures": ["Qwen3ForCausalLM"],
        "model_type": "qwen3",
        "attention_bias": False,
        "hidden_act": "silu",
        "rope_scaling": None,
        "torch_dtype": "bfloat16",
        "use_sliding_window": False,
        "sliding_window": None,
    }
    d.update(kw)
    return d


TINY_A = _base(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
               head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
               rms_norm_eps=1e-6, max_position_embeddings=128, tie_word_embeddings=True,
               bos_token_id=1, eos_token_id=2)

TINY_B = _base(num_hidden_layers=3, hidden_size=96, num_attention_heads=8, num_key_value_heads=1,
               head_dim=32, intermediate_size=160, vocab_size=384, rope_theta=1000000.0,
               rms_norm_eps=1e-5, max_position_embeddings=256, tie_word_embeddings=False,
               bos_token_id=3, eos_token_id=5)

# a window on layers 1 and 3, a head size and a vocabulary that are no power of two
TINY_C = _base(num_hidden_layers=4, hidden_size=80, num_attention_heads=6, num_key_value_heads=3,
               head_dim=48, intermediate_size=176, vocab_size=301, rope_theta=500000.0,
               rms_norm_eps=3e-6, max_position_embeddings=512, tie_word_embeddings=True,
               use_sliding_window=True, sliding_window=24,
               layer_types=["full_attention", "sliding_attention", "full_attention",
                            "sliding_attention"])

# sizes that the tensor-core kernels take (head size 64 and 128), still small
SMALL_D64 = _base(num_hidden_layers=2, hidden_size=256, num_attention_heads=8, num_key_value_heads=2,
                  head_dim=64, intermediate_size=512, vocab_size=1000, rope_theta=1000000.0,
                  rms_norm_eps=1e-6, max_position_embeddings=2048, tie_word_embeddings=False)

SMALL_D128 = _base(num_hidden_layers=2, hidden_size=384, num_attention_heads=5, num_key_value_heads=1,
                   head_dim=128, intermediate_size=640, vocab_size=1537, rope_theta=10000.0,
                   rms_norm_eps=1e-5, max_position_embeddings=4096, tie_word_embeddings=True,
                   use_sliding_window=True, sliding_window=200, max_window_layers=1)

# head size 128 with an even number of heads in q | k | v and widths that are multiples of 256: the
# kernels for many rows that fold the norms into the products and finish the heads in the q | k | v
# product's epilogue take these sizes; a window on the second layer
SMALL_E128 = _base(num_hidden_layers=3, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                   head_dim=128, intermediate_size=384, vocab_size=1201, rope_theta=250000.0,
                   rms_norm_eps=2e-6, max_position_embeddings=1024, tie_word_embeddings=False,
                   use_sliding_window=True, sliding_window=150,
                   layer_types=["full_attention", "sliding_attention", "full_attention"])

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D64": SMALL_D64, "D128": SMALL_D128, "E128": SMALL_E128}


def get(name):
    return copy.deepcopy(ALL[name])
