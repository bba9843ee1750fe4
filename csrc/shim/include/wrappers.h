// Reference-compatible umbrella for the NN modules (Linear, LayerNorm, Embedding, SelfAttention,
// MultiHeadAttention, FeedForward, TransformerBlock, GPT).
#pragma once
#include "dg_nn.h"
