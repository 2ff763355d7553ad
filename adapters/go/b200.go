// Package b200 drives libleafcutter_b200.so (C ABI in include/leafcutter_b200.h) from the Go side of LeafcutterLLM.
//
// NOT COMPILED IN THIS REPOSITORY: the build image has no Go toolchain.  This is the file a maintainer adds as
// pkg/inference/b200/b200.go (CGO_CFLAGS=-I<repo>/include, CGO_LDFLAGS=-L<dir of the library> -lleafcutter_b200).
//
// What it implements, by reference file:line
//   - inference.Model (pkg/inference/speculative.go:18-20): Model.Generate, so that SpeculativeEngine and anything else
//     written against that interface runs on the GPU path.
//   - server.ModelRunner (pkg/server/scheduler.go:55-60): Runner.RunBatch, one lc_forward_batch call per decode step for
//     all requests of the batch (a sequence slot per request), tokens streamed through req.OnToken, the result sent on
//     req.ResultCh.
package b200

/*
#include <stdlib.h>
#include "leafcutter_b200.h"

extern void lcGoToken(int64_t tok, void* user);
static inline lc_token_cb lc_go_token_cb(void) { return (lc_token_cb)lcGoToken; }
*/
import "C"

import (
	"context"
	"errors"
	"runtime/cgo"
	"sync"
	"time"
	"unsafe"
)

func lastError() error { return errors.New(C.GoString(C.lc_last_error())) }

// Model holds one engine handle.  Calls on one handle are serialised (the Rust server wraps its Engine in a Mutex,
// rust/src/api/mod.rs:42,50; the same rule applies here).
type Model struct {
	mu      sync.Mutex
	h       *C.lc_model
	vocab   int
	maxSeqs int
}

// Load parses a GGUF v3 file on the library side (rust/src/inference/engine.rs:18-49) and keeps every tensor on the device.
// maxSeqs is the number of sequence slots RunBatch may use at once (the scheduler's MaxBatchSize); 1 is enough for Generate.
func Load(path string, maxSeqLen, maxSeqs int) (*Model, error) {
	cpath := C.CString(path)
	defer C.free(unsafe.Pointer(cpath))
	var over C.lc_model_config
	over.max_seq_len = C.int32_t(maxSeqLen)
	over.max_seqs = C.int32_t(maxSeqs)
	var h *C.lc_model
	if rc := C.lc_model_load_gguf(cpath, &over, &h); rc != 0 {
		return nil, lastError()
	}
	var cfg C.lc_model_config
	if rc := C.lc_model_get_config(h, &cfg); rc != 0 {
		C.lc_model_destroy(h)
		return nil, lastError()
	}
	return &Model{h: h, vocab: int(cfg.vocab_size), maxSeqs: int(cfg.max_seqs)}, nil
}

func (m *Model) Close() {
	m.mu.Lock()
	defer m.mu.Unlock()
	if m.h != nil {
		C.lc_model_destroy(m.h)
		m.h = nil
	}
}

//export lcGoToken
func lcGoToken(tok C.int64_t, user unsafe.Pointer) {
	h := *(*cgo.Handle)(user)
	if f, ok := h.Value().(func(int)); ok && f != nil {
		f(int(tok))
	}
}

// Generate implements inference.Model: greedy decoding of up to maxTokens tokens after the prompt, stopping after token
// id 2 as Engine::generate does (rust/src/inference/engine.rs:60-63,70-72).  ctx is checked before the call; a running
// generation is not interrupted (the reference's engine has no cancellation either).
func (m *Model) Generate(ctx context.Context, prompt []int, maxTokens int, onToken func(int)) ([]int, error) {
	if err := ctx.Err(); err != nil {
		return nil, err
	}
	if len(prompt) == 0 || maxTokens <= 0 {
		return nil, errors.New("b200: empty prompt or non-positive maxTokens")
	}
	m.mu.Lock()
	defer m.mu.Unlock()
	toks := make([]C.int64_t, len(prompt))
	for i, t := range prompt {
		toks[i] = C.int64_t(t)
	}
	out := make([]C.int64_t, maxTokens)
	var n C.int32_t
	var cb C.lc_token_cb
	var user unsafe.Pointer
	if onToken != nil {
		handle := cgo.NewHandle(onToken)
		defer handle.Delete()
		cb = C.lc_go_token_cb()
		user = unsafe.Pointer(&handle)
	}
	rc := C.lc_generate(m.h, &toks[0], C.int32_t(len(toks)), C.int32_t(maxTokens), 0, 1, 1, &out[0], &n, cb, user)
	if rc != 0 {
		return nil, lastError()
	}
	res := make([]int, int(n))
	for i := range res {
		res[i] = int(out[i])
	}
	return res, nil
}

// ── server.ModelRunner ────────────────────────────────────────────────────────────────────────────────────────────────

// The request and batch types of pkg/server/scheduler.go:24-52, restated so that this file stands alone; inside the
// reference tree use server.InferRequest / server.InferResponse / server.Batch instead.
type InferRequest struct {
	ID          string
	Prompt      []int
	MaxTokens   int
	Temperature float32
	OnToken     func(int)
	ResultCh    chan InferResponse
}
type InferResponse struct {
	ID     string
	Tokens []int
	Err    error
	Took   time.Duration
}
type Batch struct{ Requests []*InferRequest }

// Runner implements server.ModelRunner over one Model with as many sequence slots as the scheduler's MaxBatchSize.
type Runner struct{ M *Model }

// RunBatch prefills every request into its own sequence slot (one lc_forward_batch call, ragged), then advances all live
// requests together, one lc_forward_batch call per decode step, until each has its MaxTokens or produced token id 2.
// Every token goes to req.OnToken as it is made; the final InferResponse goes to req.ResultCh.
func (r *Runner) RunBatch(ctx context.Context, batch *Batch) error {
	m := r.M
	n := len(batch.Requests)
	if n == 0 {
		return nil
	}
	if n > m.maxSeqs {
		return errors.New("b200: batch larger than the model's sequence slots")
	}
	m.mu.Lock()
	defer m.mu.Unlock()
	start := time.Now()
	fail := func(err error) error {
		for _, req := range batch.Requests {
			req.ResultCh <- InferResponse{ID: req.ID, Err: err, Took: time.Since(start)}
		}
		return err
	}
	if rc := C.lc_kv_clear(m.h, -1); rc != 0 {
		return fail(lastError())
	}
	seq := make([]C.int32_t, n)
	counts := make([]C.int32_t, n)
	var flat []C.int64_t
	for i, req := range batch.Requests {
		if len(req.Prompt) == 0 {
			return fail(errors.New("b200: empty prompt in batch"))
		}
		seq[i] = C.int32_t(i)
		counts[i] = C.int32_t(len(req.Prompt))
		for _, t := range req.Prompt {
			flat = append(flat, C.int64_t(t))
		}
	}
	next := make([]C.int64_t, n)
	if rc := C.lc_forward_batch(m.h, C.int32_t(n), &seq[0], &flat[0], &counts[0], nil, &next[0]); rc != 0 {
		return fail(lastError())
	}
	out := make([][]int, n)
	live := make([]int, 0, n) // indices into batch.Requests that still decode
	emit := func(i int, tok int) bool {
		req := batch.Requests[i]
		out[i] = append(out[i], tok)
		if req.OnToken != nil {
			req.OnToken(tok)
		}
		return tok != 2 && len(out[i]) < req.MaxTokens
	}
	for i := 0; i < n; i++ {
		if emit(i, int(next[i])) {
			live = append(live, i)
		}
	}
	for len(live) > 0 {
		if err := ctx.Err(); err != nil {
			return fail(err)
		}
		k := len(live)
		ids := make([]C.int32_t, k)
		toks := make([]C.int64_t, k)
		ones := make([]C.int32_t, k)
		for j, i := range live {
			ids[j] = C.int32_t(i)
			toks[j] = C.int64_t(out[i][len(out[i])-1])
			ones[j] = 1
		}
		step := make([]C.int64_t, k)
		if rc := C.lc_forward_batch(m.h, C.int32_t(k), &ids[0], &toks[0], &ones[0], nil, &step[0]); rc != 0 {
			return fail(lastError())
		}
		still := live[:0]
		for j, i := range live {
			if emit(i, int(step[j])) {
				still = append(still, i)
			}
		}
		live = still
	}
	for i, req := range batch.Requests {
		req.ResultCh <- InferResponse{ID: req.ID, Tokens: out[i], Took: time.Since(start)}
	}
	return nil
}
