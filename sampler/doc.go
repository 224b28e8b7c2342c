// Package sampler binds libborn_sampler.so, the B200 (sm_100a) token-sampling and
// constrained-decoding library, into born.
//
// UNCOMPILED: the image this repository was built in has no Go toolchain.  The C ABI these
// files bind (include/born_sampler.h) is exercised by the Python mirror born_b200/sampler.py;
// these files are that mirror written in the reference's own language, ready for a
// maintainer to build.
//
// Layout follows born v0.1.1: the implementation would live in internal/sampler and be
// re-exported from sampler/ by type aliases, as nn/nn.go does for internal/nn.  Idioms kept
// from the reference:
//   - a plain config struct whose zero values mean "off" (internal/optim/adam.go:59-91);
//   - optional backend capabilities are extra methods found by type assertion
//     (internal/nn/activation.go:7-20,41-52): SamplerBackend below;
//   - programmer errors panic (internal/backend/cpu/backend.go:35-37), runtime failures
//     come back as error (internal/tensor/raw.go:89-92);
//   - greedy selection is the reference's argmax: the first maximum wins
//     (internal/nn/cross_entropy.go:241-251).
//
// Two loaders implement the same unexported `binding` interface: cgo.go (build tag cgo) and
// purego.go (no cgo, dlopen + register trampolines; keeps the reference's "no CGO" build).
package sampler
