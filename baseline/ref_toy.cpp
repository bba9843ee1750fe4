// Timing harness for the UNMODIFIED reference headers (compiled against baseline/_ref/src).
// Configuration 2: decoder with vocab 256, d_model 64, 2 layers, 4 heads, FFN 256 (the
// reference's FeedForward is always 4*d_model), sequence 32, batch 8, fp32, Adam 3e-4, uniform
// random tokens, next-token cross-entropy. The reference's GPT::forward handles one sequence
// per call, so a batch is 8 forward calls whose losses are added before one backward.
// Prints: ms_per_step tokens_per_s first_loss last_loss
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include "dummy.h"

int main(int argc, char** argv) {
  int steps = argc > 1 ? std::atoi(argv[1]) : 5;
  int warmup = argc > 2 ? std::atoi(argv[2]) : 1;
  const int V = 256, S = 32, D = 64, H = 4, Lyr = 2, B = 8;
  manual_seed(0);
  GPT model(V, S, D, H, Lyr);
  Adam opt(3e-4f);
  auto params = model.parameters();
  std::mt19937 rng(1);
  std::uniform_int_distribution<int> tok(0, V - 1);
  auto pos = std::make_shared<Tensor>(std::vector<int>{S}, false);
  for (int i = 0; i < S; ++i) pos->data_ptr()[i] = (float)i;
  std::vector<std::shared_ptr<Tensor>> ids(B), tgt(B);
  for (int b = 0; b < B; ++b) {
    ids[b] = std::make_shared<Tensor>(std::vector<int>{S}, false);
    tgt[b] = std::make_shared<Tensor>(std::vector<int>{S, V}, false);
    for (int i = 0; i < S; ++i) {
      ids[b]->data_ptr()[i] = (float)tok(rng);
      tgt[b]->data_ptr()[i * V + tok(rng)] = 1.0f;
    }
  }
  float first = 0.f, last = 0.f;
  std::chrono::steady_clock::time_point t0;
  for (int step = 0; step < warmup + steps; ++step) {
    if (step == warmup) t0 = std::chrono::steady_clock::now();
    for (auto& p : params) p->zero_grad();
    std::shared_ptr<Tensor> total;
    for (int b = 0; b < B; ++b) {
      auto loss = cross_entropy(softmax(model.forward(ids[b], pos)), tgt[b]);
      total = total ? add(total, loss) : loss;
    }
    last = total->data_at(0) / B;
    if (step == 0) first = last;
    total->backward();
    for (auto& p : params) opt.step(p);
  }
  double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / steps;
  std::printf("%.4f %.2f %g %g\n", ms, B * S / (ms / 1e3), first, last);
  return 0;
}
