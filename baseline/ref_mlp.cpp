// Timing harness for the UNMODIFIED reference headers (compiled against baseline/_ref/src).
// Configuration 1: fp32 MLP 784 -> 128 ReLU -> 10, batch 64, N(0,1) inputs, uniform labels,
// softmax cross-entropy, SGD 1e-2, seed 0. The reference's models/mlp.cpp is empty, so the model
// is composed from its Linear, relu, softmax, cross_entropy and SGD.
// Prints: ms_per_step samples_per_s first_loss last_loss
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include "dummy.h"

int main(int argc, char** argv) {
  int steps = argc > 1 ? std::atoi(argv[1]) : 100;
  int warmup = argc > 2 ? std::atoi(argv[2]) : 3;
  manual_seed(0);
  Linear fc1(784, 128), fc2(128, 10);
  auto x = randn({64, 784});
  x->requires_grad = false;
  auto y = std::make_shared<Tensor>(std::vector<int>{64, 10}, false);
  std::mt19937 rng(0);
  std::uniform_int_distribution<int> lab(0, 9);
  for (int i = 0; i < 64; ++i) y->data_ptr()[i * 10 + lab(rng)] = 1.0f;
  std::vector<std::shared_ptr<Tensor>> params = {fc1.W, fc1.b, fc2.W, fc2.b};
  float first = 0.f, last = 0.f;
  std::chrono::steady_clock::time_point t0;
  for (int step = 0; step < warmup + steps; ++step) {
    if (step == warmup) t0 = std::chrono::steady_clock::now();
    for (auto& p : params) p->zero_grad();
    auto loss = cross_entropy(softmax(fc2.forward(relu(fc1.forward(x)))), y);
    last = loss->data_at(0);
    if (step == 0) first = last;
    loss->backward();
    for (auto& p : params) SGD(p, 1e-2f);
  }
  double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / steps;
  std::printf("%.4f %.2f %g %g\n", ms, 64 / (ms / 1e3), first, last);
  return 0;
}
