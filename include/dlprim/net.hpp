// Net: a static graph of operators described by JSON, executed in file order on one stream.
// Inference subset of the reference's Net (include/dlprim/net.hpp:21-317, src/net.cpp): JSON loading,
// operator wiring by tensor name, in-place and alias operators, parameter naming, one shared
// workspace, liveness-based reuse of activation memory, forward.  There is no backward here.
//
// Two inference-only additions that do not change results beyond rounding:
//  * an execution plan that folds `Convolution2D -> Elementwise(sum)` (the residual add of ResNet
//    blocks) into the convolution's epilogue, so the sum never makes its own pass over memory;
//  * replay of the whole forward pass as one CUDA graph.
// Both can be switched off; keep_intermediate_tensors(true) switches the first one off as well,
// because then every named tensor must hold its own value after forward().
#pragma once
#include <dlprim/operator.hpp>
#include <map>
#include <string>
#include <vector>

typedef struct CUgraphExec_st *cudaGraphExec_t;

namespace dlprim {

class DLPRIM_API Net {
public:
    Net(Context &ctx);
    ~Net();
    Net(Net const &) = delete;
    Net const &operator=(Net const &) = delete;

        /// The activation merge of the reference's ONNX importer (src/importers/onnx.cpp:531-579), as a pass over a
        /// network description that is already JSON: an Activation operator that directly follows a Convolution2D,
        /// InnerProduct or Elementwise operator whose own activation is "identity", consumes that operator's output
        /// and is its only consumer (the tensor is not a network output either) disappears into the operator's
        /// "activation" option, and the operator writes the activation's output tensor.  Returns the number merged.
        static int merge_activations(json::value &network);

    void load_from_json(json::value const &v);
    void load_from_json_file(std::string const &name);
    void add_input_tensor(std::string const &name, TensorSpecs const &ts, bool requires_gradient = false);
    void mark_output_tensor(std::string const &name);
    void add_operator(std::unique_ptr<Operator> op, std::string const &name, std::vector<std::string> const &inputs,
                      std::vector<std::string> const &outputs, std::vector<std::string> const &parameters = std::vector<std::string>(),
                      bool frozen = false);

    /// Only CalculationsMode::predict is available on this path.
    void mode(CalculationsMode mode);
    CalculationsMode mode() const { return mode_; }
    bool keep_intermediate_tensors() const { return keep_intermediate_tensors_; }
    void keep_intermediate_tensors(bool keep) { keep_intermediate_tensors_ = keep; }
    /// Fold residual sums into the producing convolution (default on).
    void fuse_operators(bool v) { fuse_ = v; }
    /// Replay forward() as a CUDA graph from the second call on (default on).
    void use_cuda_graph(bool v) { use_graph_ = v; drop_graph(); }
    /// Run a convolution that does not depend on the operators just before it (the projection shortcut of a residual
    /// block) on a second stream, from the point where its inputs are ready to the point where its result is first used.
    /// Takes effect at the next setup().  Default off.
    void concurrent_branches(bool v) { side_branches_ = v; }
    bool concurrent_branches() const { return side_branches_; }

    /// Allocate tensors, parameters and the workspace; build the execution plan.
    void setup();
    /// Propagate the input tensors' current shapes through the operators and re-allocate.
    void reshape();
    /// Change the shape of an input tensor; call reshape() afterwards.
    void reshape_input(std::string const &name, Shape const &s);

    /// Parameter files in the reference's "DLPW" container (src/net.cpp:63-101,204-305).
    void load_parameters(std::istream &s, bool allow_missing = false);
    void load_parameters(std::string const &file_name, bool allow_missing = false);
    void save_parameters(std::string const &file_name);
    /// Upload the host copies of all parameters; operators re-pack their weights on the next forward.
    void copy_parameters_to_device();
    void copy_parameters_to_host();

    std::map<std::string, Tensor> &tensors() { return tensors_; }
    std::map<std::string, Tensor> &params() { return parameters_; }
    Tensor &tensor(std::string const &name);
    Tensor &param(std::string const &name);
    std::vector<std::string> const &input_names() { return inputs_; }
    std::vector<std::string> const &output_names() { return outputs_; }
    Tensor &input(unsigned id);
    Tensor &output(unsigned id);

    void forward(ExecutionContext const &ectx, bool sync = false);

    /// One line per step of the execution plan: "<operator name> <type> <kernel> [fused with ...]".
    std::vector<std::string> describe_plan() const;
    /// Bytes of device memory holding activations (after reuse) and the peak without reuse.
    size_t activation_memory() const { return activation_bytes_; }
    size_t activation_memory_without_reuse() const { return activation_bytes_naive_; }

private:
    struct Connection {
        std::string name;
        std::unique_ptr<Operator> op;
        std::vector<std::string> input_names, output_names, parameter_names;
        std::vector<TensorSpecs> input_specs, output_specs, parameter_specs;
        std::vector<Tensor> input_tensors, output_tensors, parameters;
        size_t ws_size = 0;
    };
    struct Step {
        enum Kind { plain, conv_residual } kind = plain;
        unsigned conn = 0;          // the operator that runs
        unsigned fused_conn = 0;    // conv_residual: the Elementwise it absorbs
        std::string residual;       // conv_residual: tensor added to the convolution result
        std::string result;         // conv_residual: tensor the sum is written to
        float residual_scale = 1.0f;
        StandardActivations post_activation = StandardActivations::identity;
        std::vector<std::string> reads, writes;
        // concurrent branches: this step runs on the second stream, launched before step fork_at and joined before step join_at
        int fork_at = -1, join_at = -1;
    };
    void build_plan();
    void allocate_tensors();
    void allocate_parameters();
    void bind_tensors();
    void run_steps(ExecutionContext const &e);
    void drop_graph();
    std::string root_of(std::string const &name) const;

    Context ctx_;
    CalculationsMode mode_ = CalculationsMode::predict;
    bool keep_intermediate_tensors_ = false;
    bool fuse_ = true, use_graph_ = true;
    bool side_branches_ = false;
    bool is_setup_ = false;

    std::map<std::string, TensorSpecs> tensor_specs_;
    std::map<std::string, TensorSpecs> parameter_specs_;
    std::map<std::string, std::string> alias_sources_;   // alias tensor -> tensor whose memory it shares
    std::vector<Connection> connections_;
    std::map<std::string, unsigned> connections_index_;
    std::vector<Step> steps_;
    std::vector<std::string> inputs_, outputs_;

    Tensor workspace_;
    Tensor side_workspace_;      // for the steps on the second stream
    Tensor pool_;
    std::map<std::string, Tensor> tensors_;
    std::map<std::string, Tensor> parameters_;
    size_t activation_bytes_ = 0, activation_bytes_naive_ = 0;

    cudaGraphExec_t graph_exec_ = nullptr;
    cudaStream_t graph_stream_ = nullptr;
    cudaStream_t side_stream_ = nullptr;
    std::vector<cudaEvent_t> side_events_;   // two per step on the second stream: inputs ready, result ready
    int forwards_since_change_ = 0;
};

} // namespace dlprim
