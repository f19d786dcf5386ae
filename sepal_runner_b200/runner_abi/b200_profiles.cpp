// The profiles of libsepal_runner_b200.so: what makes this library's kernels reachable through the reference's C ABI.
//
// A backend library of the reference is its c_api.cpp object code plus a sepal::register_backend_profiles() of the backend's own
// (runner/include/sepal/engine.hpp:1-17,42-59; the CUDA library's is runner/cuda/src/gpu_profiles.cpp:10-54). This file is that
// function for the B200 kernels. The Makefile beside it compiles the reference's c_api.cpp, registry.cpp and core sources where
// they lie, unmodified, and links them with this file and cuda_gemm_b200.cu: sepal_open / sepal_score / sepal_info / sepal_close,
// the option parsing, the unknown-key refusal and the error path are the reference's object code.
//
// Profiles
//   gpu-b200-f16   every projection of the trunk is multiplied by sepal_b200_gemm_f16 (binary16 operands rounded once, float32
//                  accumulation), reached through the reference's own provider interface: the trunk is the reference's row
//                  executor (sepal::ref::run_rows, runner/include/sepal/ref/executor.hpp:201), which sends every matrix multiply
//                  to the sepal::GemmProvider it is given; here that provider is sepal::cuda::CudaGemm as cuda_gemm_b200.cu
//                  implements it. Attention, the delta rule, the norms and the Clef head are the reference's host code: they are
//                  outside this library's path. It is the drop-in that proves the boundary (any geometry, the reference's own
//                  fixtures), not the fast engine: that is sepal_b200_trunk_* (include/sepal_b200.h).
//   cpu-ref, cpu-ref64   the reference's oracle engines, registered as its CPU library registers them, so that one library answers
//                  both sides of a comparison.
// Extra option keys of gpu-b200-f16: "arena_mib" (the provider's single device allocation; default 2048).
#include <chrono>
#include <numeric>

#include "sepal/clef_head.hpp"
#include "sepal/cuda/cuda_gemm.hpp"
#include "sepal/engine.hpp"
#include "sepal/ref/executor.hpp"
#include "sepal/trained_model.hpp"

namespace sepal {

namespace {

void head_embedding_row(const void* model, std::uint32_t token, float* out) { static_cast<const TrainedModel*>(model)->embedding_row(token, out); }

class B200Engine final : public DecisionEngine {
public:
    B200Engine(TrainedModel model, const EngineOptions& options, std::size_t arena_bytes)
        : model_(std::move(model)), weights_(model_.merged_weights<float>()),
          gemm_(cuda::CudaGemmOptions{options.device, cuda::Precision::F16, arena_bytes, 0}), max_tokens_(options.max_tokens) {}

    std::vector<RequestLogits> score(std::span<const EncodedRequest> requests) override {
        using Clock = std::chrono::steady_clock;
        const auto ms = [](Clock::time_point from) { return std::chrono::duration<double, std::milli>(Clock::now() - from).count(); };
        const Clock::time_point begun = Clock::now();
        for (const EncodedRequest& r : requests) {  // everything is checked before any work, as decision.hpp asks
            check_request(r, model_.config().vocab_size);
            if (r.token_ids.size() > max_tokens_)
                throw std::invalid_argument("request has " + std::to_string(r.token_ids.size()) + " tokens, the limit is " + std::to_string(max_tokens_));
        }
        times_ = {};
        std::vector<RequestLogits> out;
        out.reserve(requests.size());
        for (const EncodedRequest& r : requests) {
            const Clock::time_point trunk_begun = Clock::now();
            ref::Row<float> row;
            row.token_ids = r.token_ids;
            row.readout_offsets.resize(r.token_ids.size());  // the head reads spans anywhere in the sequence: every position's final state
            std::iota(row.readout_offsets.begin(), row.readout_offsets.end(), std::size_t{0});
            std::vector<ref::Row<float>> rows;
            rows.push_back(std::move(row));
            const std::vector<ref::RowResult<float>> result = ref::run_rows<float>(gemm_, model_.config(), weights_, rows);
            const std::vector<float> hidden(result[0].hidden.data(), result[0].hidden.data() + result[0].hidden.size());
            times_.trunk_ms += ms(trunk_begun);
            times_.tokens += r.token_ids.size();
            const Clock::time_point head_begun = Clock::now();
            out.push_back(clef_head_reference(model_.head(), hidden, r, &head_embedding_row, &model_));
            times_.head_ms += ms(head_begun);
        }
        times_.total_ms = ms(begun);
        return out;
    }

    std::string profile() const override { return "gpu-b200-f16"; }
    std::uint64_t max_tokens() const override { return max_tokens_; }
    std::uint64_t hidden_size() const override { return model_.config().hidden_size; }
    std::string runtime() const override {
        const cuda::DeviceInfo d = gemm_.device_info();
        return "projections on " + d.name + " (sm_" + std::to_string(d.compute_major) + std::to_string(d.compute_minor) +
               ") by sepal_b200_gemm_f16 behind sepal::GemmProvider; mixers, norms and head on the host (reference executor)";
    }
    ScoreTimes last_times() const override { return times_; }

private:
    TrainedModel model_;
    Weights<float> weights_;
    cuda::CudaGemm gemm_;
    std::uint64_t max_tokens_;
    ScoreTimes times_;
};

std::unique_ptr<DecisionEngine> make_b200(const EngineOptions& o) {
    if (o.max_tokens == 0) throw std::invalid_argument("max_tokens must be positive");
    std::size_t arena_mib = 2048;
    if (const auto it = o.extra.find("arena_mib"); it != o.extra.end()) arena_mib = static_cast<std::size_t>(it->second.as_uint());
    if (arena_mib == 0) throw std::invalid_argument("arena_mib must be positive");
    TrainedModel model = TrainedModel::open(o.final_dir, o.base_dir);
    return std::make_unique<B200Engine>(std::move(model), o, arena_mib << 20);
}

}  // namespace

void register_backend_profiles() {
    register_ref_profiles();
    register_profile({"gpu-b200-f16", "cuda", {"arena_mib"}, [](const EngineOptions& o) { return make_b200(o); }});
}

}  // namespace sepal
