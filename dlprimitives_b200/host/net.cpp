// Net: graph loading, wiring, memory planning, execution plan, forward.
#include <dlprim/net.hpp>
#include <dlprim/json.hpp>
#include <dlprim/ops/conv2d.hpp>
#include <dlprim/ops/inner_product.hpp>
#include <dlprim/ops/glue.hpp>
#include "host_util.hpp"

#include <cuda_runtime.h>
#include <algorithm>
#include <cstring>
#include <fstream>
#include <set>
#include <sstream>

namespace dlprim {
using host::cuda_check;

Net::Net(Context &ctx) : ctx_(ctx) {}
Net::~Net()
{
    drop_graph();
    for(cudaEvent_t ev : side_events_) cudaEventDestroy(ev);
    if(side_stream_) cudaStreamDestroy(side_stream_);
}

void Net::mode(CalculationsMode m)
{
    if(m != CalculationsMode::predict) throw NotImplementedError("only CalculationsMode::predict is available: this library has no backward pass");
    mode_ = m;
}

// -------------------------------------------------------------------------------------------- building
void Net::load_from_json(json::value const &v)
{
    for(json::value const &input : v["inputs"].array()) {
        std::vector<int> dims = input.get<std::vector<int> >("shape");
        Shape sp = Shape::from_range(dims.begin(), dims.end());
        DataType dt = string_to_data_type(input.get("dtype", "float"));
        add_input_tensor(input.get("name", "data"), TensorSpecs(sp, dt));
    }
    json::value empty_options = json::object();
    for(json::value const &op : v["operators"].array()) {
        std::string name = op.get<std::string>("name");
        std::string type = op.get<std::string>("type");
        bool frozen = op.get("frozen", false);
        std::vector<std::string> inputs = op.get("inputs", std::vector<std::string>());
        std::vector<std::string> outputs = op.get("outputs", std::vector<std::string>());
        std::vector<std::string> params = op.get("params", std::vector<std::string>());
        json::value const &opts = op.find("options").is_undefined() ? empty_options : op["options"];
        std::unique_ptr<Operator> oper = create_by_name(ctx_, type, opts);
        add_operator(std::move(oper), name, inputs, outputs, params, frozen);
    }
    for(json::value const &output : v["outputs"].array()) {
        if(output.type() == json::is_string) mark_output_tensor(output.str());
        else mark_output_tensor(output.get<std::string>("name"));
    }
}

int Net::merge_activations(json::value &network)
{
    json::array &src = network["operators"].array();
    // every consumer of a tensor name, over the whole description, and the network's outputs
    std::map<std::string, int> uses;
    for(json::value const &op : src)
        for(std::string const &in : op.get("inputs", std::vector<std::string>())) uses[in]++;
    std::set<std::string> net_outputs;
    for(json::value const &o : network["outputs"].array()) net_outputs.insert(o.type() == json::is_string ? o.str() : o.get<std::string>("name"));
    json::array kept;
    int merged = 0;
    for(json::value const &op : src) {
        bool merge = false;
        if(op.get<std::string>("type") == "Activation" && !kept.empty()) {
            json::value &prev = kept.back();                      // "directly follows": the operator kept last
            std::string type = prev.get<std::string>("type");
            std::vector<std::string> prev_out = prev.get("outputs", std::vector<std::string>());
            std::vector<std::string> in = op.get("inputs", std::vector<std::string>());
            std::vector<std::string> out = op.get("outputs", std::vector<std::string>());
            merge = (type == "Convolution2D" || type == "InnerProduct" || type == "Elementwise") && in.size() == 1 && out.size() == 1
                    && prev_out.size() == 1 && prev_out[0] == in[0] && prev.get("options.activation", "identity") == "identity"
                    && uses[in[0]] == 1 && !net_outputs.count(in[0]);
            if(merge) {
                prev["outputs"].array()[0] = json::value(out[0]);
                prev["options"]["activation"] = json::value(op.get("options.activation", "identity"));
                merged++;
            }
        }
        if(!merge) kept.push_back(op);
    }
    src = kept;
    return merged;
}

void Net::load_from_json_file(std::string const &name)
{
    std::ifstream f(name);
    if(!f) throw ValidationError("Failed to open file " + name);
    json::value net;
    int line = -1;
    if(!net.load(f, true, &line)) throw ValidationError("Failed to load json from " + name + ", syntax error at line " + std::to_string(line));
    load_from_json(net);
}

void Net::add_input_tensor(std::string const &name, TensorSpecs const &ts, bool)
{
    if(tensor_specs_.count(name)) throw ValidationError("Tensor " + name + " already exists");
    tensor_specs_[name] = ts;
    inputs_.push_back(name);
    is_setup_ = false;
}

void Net::mark_output_tensor(std::string const &name)
{
    if(!tensor_specs_.count(name)) throw ValidationError("mark_output_tensor::No such tensor name " + name);
    if(std::find(outputs_.begin(), outputs_.end(), name) == outputs_.end()) outputs_.push_back(name);
    is_setup_ = false;
}

void Net::add_operator(std::unique_ptr<Operator> op, std::string const &name, std::vector<std::string> const &inputs,
                       std::vector<std::string> const &outputs, std::vector<std::string> const &parameters, bool)
{
    if(connections_index_.count(name)) throw ValidationError("Operator with name " + name + " exists");
    Connection conn;
    conn.name = name;
    conn.input_names = inputs;
    conn.output_names = outputs;
    for(std::string const &in : inputs) {
        auto p = tensor_specs_.find(in);
        if(p == tensor_specs_.end()) throw ValidationError("No such tensor " + in + " for operator " + name);
        conn.input_specs.push_back(p->second);
    }
    op->mode(mode_);
    op->cache_packed_parameters(true);
    op->setup(conn.input_specs, conn.output_specs, conn.parameter_specs, conn.ws_size);
    if(conn.output_specs.size() != outputs.size())
        throw ValidationError("Operator " + name + " expects " + std::to_string(conn.output_specs.size()) + " outputs, got "
                              + std::to_string(outputs.size()));
    if(op->alias_generator()) {
        DLPRIM_CHECK(inputs.size() == outputs.size());
        for(size_t i = 0; i < inputs.size(); i++) {
            if(inputs[i] != outputs[i] && tensor_specs_.count(outputs[i])) throw ValidationError("Tensor " + outputs[i] + " already exists");
            if(inputs[i] != outputs[i]) alias_sources_[outputs[i]] = inputs[i];
            tensor_specs_[outputs[i]] = conn.output_specs[i];
        }
    }
    else {
        for(size_t i = 0; i < outputs.size(); i++) {
            auto p = tensor_specs_.find(outputs[i]);
            if(p == tensor_specs_.end()) {
                tensor_specs_[outputs[i]] = conn.output_specs[i];
                continue;
            }
            // an existing name is allowed only for an in-place operator: the output is one of its inputs
            if(std::find(inputs.begin(), inputs.end(), outputs[i]) == inputs.end())
                throw ValidationError("Tensor " + outputs[i] + " already exists and is not an input of " + name);
            if(p->second != conn.output_specs[i]) {
                std::ostringstream ss;
                ss << "Tensor " << outputs[i] << " is used in place by " << name << " with different specs " << p->second << " vs "
                   << conn.output_specs[i];
                throw ValidationError(ss.str());
            }
        }
    }
    unsigned params_no = unsigned(conn.parameter_specs.size());
    if(params_no < parameters.size())
        throw ValidationError("Too many parameter names for operaror " + name + " expecting " + std::to_string(params_no) + " got "
                              + std::to_string(parameters.size()));
    conn.parameter_names = parameters;
    conn.parameter_names.resize(params_no);
    for(size_t i = 0; i < conn.parameter_names.size(); i++) {
        std::string &pname = conn.parameter_names[i];
        if(pname.empty() || pname == "auto") pname = name + "." + std::to_string(i);
        auto p = parameter_specs_.find(pname);
        if(p == parameter_specs_.end()) parameter_specs_[pname] = conn.parameter_specs[i];
        else if(p->second != conn.parameter_specs[i]) {
            std::ostringstream ss;
            ss << "Conflicting requirements for parameters specifications " << p->second << " vs " << conn.parameter_specs[i] << " for " << pname;
            throw ValidationError(ss.str());
        }
    }
    conn.op = std::move(op);
    connections_index_[name] = unsigned(connections_.size());
    connections_.push_back(std::move(conn));
    is_setup_ = false;
}

// -------------------------------------------------------------------------------------------- plan
std::string Net::root_of(std::string const &name) const
{
    std::string cur = name;
    for(auto p = alias_sources_.find(cur); p != alias_sources_.end(); p = alias_sources_.find(cur)) cur = p->second;
    return cur;
}

void Net::build_plan()
{
    steps_.clear();
    // consumers of every tensor name, by connection index
    std::map<std::string, std::vector<unsigned> > consumers;
    for(unsigned i = 0; i < connections_.size(); i++)
        for(std::string const &n : connections_[i].input_names) consumers[n].push_back(i);
    std::set<std::string> outputs(outputs_.begin(), outputs_.end());
    std::vector<int> absorbed_by(connections_.size(), -1);   // Elementwise -> convolution that absorbs it
    std::vector<int> absorbs(connections_.size(), -1);

    if(fuse_ && !keep_intermediate_tensors_) {
        for(unsigned j = 0; j < connections_.size(); j++) {
            Connection &add = connections_[j];
            Elementwise *ew = dynamic_cast<Elementwise *>(add.op.get());
            if(!ew || ew->config().op != Elementwise::Config::elementwise_sum) continue;
            if(add.input_names.size() != 2 || add.input_names[0] == add.input_names[1]) continue;
            // The operand written last before the sum must come from a convolution that feeds nothing else.  "Written
            // last" counts every writer of the tensor's storage (in-place operators rewrite a name, aliases share it).
            auto last_writer = [&](std::string const &name) {
                const std::string root = root_of(name);
                for(int m = int(j) - 1; m >= 0; m--)
                    for(std::string const &o : connections_[m].output_names)
                        if(root_of(o) == root) return m;
                return -1;
            };
            const int w0 = last_writer(add.input_names[0]), w1 = last_writer(add.input_names[1]);
            if(w0 < 0 && w1 < 0) continue;
            if(w0 == w1) continue;                         // both operands in one storage
            const int pick = w0 > w1 ? 0 : 1;
            const unsigned best = unsigned(std::max(w0, w1));
            std::string const &t = add.input_names[pick];
            std::string const &other = add.input_names[1 - pick];
            Connection &cv = connections_[best];
            Convolution2D *conv = dynamic_cast<Convolution2D *>(cv.op.get());
            if(!conv || absorbs[best] >= 0) continue;
            if(cv.output_names.size() != 1 || cv.output_names[0] != t) continue;
            if(std::find(cv.input_names.begin(), cv.input_names.end(), t) != cv.input_names.end()) continue;
            if(consumers[t].size() != 1 || outputs.count(t) || alias_sources_.count(t)) continue;
            bool aliased = false;
            for(auto const &a : alias_sources_) aliased = aliased || a.second == t;
            if(aliased) continue;
            if(ew->config().coeff[pick] != 1.0f) continue;
            if(std::string(conv->algo()) == "depthwise_separable") continue;
            // The fusion moves the write of the sum's output forward to the convolution's step.  So between the
            // two nothing may write the other operand, and nothing may read or write the storage of the sum's
            // output: with an in-place sum (output == other operand) a reader of the shortcut in between would
            // otherwise see shortcut + branch instead of the shortcut.
            bool clobbered = false;
            const std::string result_root = root_of(add.output_names[0]), other_root = root_of(other);
            for(unsigned m = best + 1; m < j && !clobbered; m++) {
                for(std::string const &o : connections_[m].output_names)
                    clobbered = clobbered || root_of(o) == other_root || root_of(o) == result_root;
                for(std::string const &in : connections_[m].input_names)
                    clobbered = clobbered || root_of(in) == result_root;
            }
            // the convolution itself must not read the storage it would now overwrite
            for(std::string const &in : cv.input_names) clobbered = clobbered || root_of(in) == result_root;
            if(clobbered) continue;
            absorbs[best] = int(j);
            absorbed_by[j] = int(best);
        }
    }

    for(unsigned i = 0; i < connections_.size(); i++) {
        if(absorbed_by[i] >= 0) continue;
        Connection &c = connections_[i];
        Step st;
        st.conn = i;
        if(absorbs[i] >= 0) {
            Connection &add = connections_[absorbs[i]];
            Elementwise *ew = static_cast<Elementwise *>(add.op.get());
            int pick = add.input_names[0] == c.output_names[0] ? 0 : 1;
            st.kind = Step::conv_residual;
            st.fused_conn = unsigned(absorbs[i]);
            st.residual = add.input_names[1 - pick];
            st.result = add.output_names[0];
            st.residual_scale = ew->config().coeff[1 - pick];
            st.post_activation = ew->config().activation;
            st.reads = c.input_names;
            st.reads.push_back(st.residual);
            st.writes = {st.result};
        }
        else {
            st.reads = c.input_names;
            st.writes = c.output_names;
        }
        steps_.push_back(st);
    }

    // Concurrent branches: a plain convolution whose inputs were complete well before its turn (nothing between their last
    // writer and the convolution writes them or touches its output's storage) is launched on the second stream as soon
    // as those inputs are ready and joined before the first step that touches its result.
    if(side_branches_ && !keep_intermediate_tensors_) {
        auto roots = [&](std::vector<std::string> const &names) {
            std::set<std::string> r;
            for(std::string const &n : names) r.insert(root_of(n));
            return r;
        };
        auto touches = [&](Step const &st, std::set<std::string> const &rs, bool reads_too) {
            for(std::string const &n : st.writes) if(rs.count(root_of(n))) return true;
            if(reads_too) for(std::string const &n : st.reads) if(rs.count(root_of(n))) return true;
            return false;
        };
        int busy_until = -1;                       // one branch at a time on the second stream
        for(int s = 0; s < int(steps_.size()); s++) {
            Step &st = steps_[s];
            if(st.kind != Step::plain || !dynamic_cast<Convolution2D *>(connections_[st.conn].op.get())) continue;
            const std::set<std::string> in = roots(st.reads), out = roots(st.writes);
            bool overlap = false;
            for(std::string const &r : in) overlap = overlap || out.count(r);
            if(overlap) continue;
            int w = -1;                             // last step before s that writes an input
            for(int m = s - 1; m >= 0 && w < 0; m--) if(touches(steps_[m], in, false)) w = m;
            if(w >= s - 1 || w + 1 <= busy_until) continue;
            bool ok = true;
            for(int m = w + 1; m < s && ok; m++) ok = !touches(steps_[m], out, true);
            int j = -1;                             // first step after s that touches the result
            for(int m = s + 1; m < int(steps_.size()) && j < 0; m++) {
                if(touches(steps_[m], out, true)) j = m;
                else if(touches(steps_[m], in, false)) ok = false;      // an input rewritten while the branch may still read it
            }
            if(!ok || j < 0) continue;
            for(std::string const &o : outputs_) ok = ok && !out.count(root_of(o));
            if(!ok) continue;
            st.fork_at = w + 1;
            st.join_at = j;
            busy_until = j;
        }
    }
}

// -------------------------------------------------------------------------------------------- memory
void Net::allocate_tensors()
{
    tensors_.clear();
    // liveness of every root tensor over the steps of the plan
    std::map<std::string, std::pair<int, int> > live;   // root -> [first write or -1 for inputs, last use]
    auto touch = [&](std::string const &name, int step) {
        std::string r = root_of(name);
        auto p = live.find(r);
        if(p == live.end()) live[r] = std::make_pair(step, step);
        else p->second.second = std::max(p->second.second, step);
    };
    for(std::string const &in : inputs_) touch(in, -1);
    for(int s = 0; s < int(steps_.size()); s++) {
        // a step on the second stream may write its result from its launch point on and read its inputs until it is joined
        for(Step const &side : steps_)
            if(side.fork_at == s) {
                for(std::string const &n : side.writes) { touch(n, s); touch(n, side.join_at); }
                for(std::string const &n : side.reads) touch(n, side.join_at);
            }
        for(std::string const &n : steps_[s].writes) touch(n, s);
        for(std::string const &n : steps_[s].reads) touch(n, s);
    }
    const int forever = int(steps_.size()) + 1;
    for(std::string const &in : inputs_) live[root_of(in)].second = forever;     // callers may re-read or re-fill inputs
    for(std::string const &out : outputs_) touch(out, forever);

    // bytes a root needs: the largest of its own specs and its aliases' (all share one block)
    std::map<std::string, size_t> bytes;
    for(auto const &ts : tensor_specs_) {
        std::string r = root_of(ts.first);
        if(!live.count(r)) continue;   // produced by a step that was folded away and never materialised
        bytes[r] = std::max(bytes[r], (ts.second.memory_size() + 255) / 256 * 256);
    }
    activation_bytes_naive_ = 0;
    for(auto const &b : bytes) activation_bytes_naive_ += b.second;

    // Offsets.  Without reuse every root has its own block; with reuse a block is handed to a later
    // root once the earlier one is dead (first fit over the blocks ordered by first use).
    struct Block { size_t offset, size; int busy_until; };
    std::vector<Block> blocks;
    std::map<std::string, size_t> offsets;
    std::vector<std::pair<int, std::string> > order;
    for(auto const &l : live) order.push_back(std::make_pair(l.second.first, l.first));
    std::sort(order.begin(), order.end());
    size_t total = 0;
    for(auto const &o : order) {
        std::string const &r = o.second;
        size_t need = bytes[r];
        int first = live[r].first, last = live[r].second;
        int chosen = -1;
        if(!keep_intermediate_tensors_) {
            for(size_t b = 0; b < blocks.size(); b++) {
                // strictly before: an operator never gets the block of one of its own inputs
                if(blocks[b].busy_until < first && blocks[b].size >= need && (chosen < 0 || blocks[b].size < blocks[chosen].size))
                    chosen = int(b);
            }
        }
        if(chosen < 0) {
            blocks.push_back(Block{total, need, last});
            chosen = int(blocks.size()) - 1;
            total += need;
        }
        else
            blocks[chosen].busy_until = last;
        offsets[r] = blocks[chosen].offset;
    }
    activation_bytes_ = total;
    pool_ = Tensor(ctx_, Shape(std::max<size_t>(total, 256)), uint8_data);
    for(auto const &ts : tensor_specs_) {
        std::string r = root_of(ts.first);
        auto off = offsets.find(r);
        if(off == offsets.end()) continue;
        size_t elem = size_of_data_type(ts.second.dtype());
        tensors_[ts.first] = pool_.sub_tensor(off->second / elem, ts.second.shape(), ts.second.dtype());
    }
}

void Net::allocate_parameters()
{
    // keep existing parameter tensors (and their values) when the specs did not change
    std::map<std::string, Tensor> old;
    old.swap(parameters_);
    for(auto const &ps : parameter_specs_) {
        auto p = old.find(ps.first);
        if(p != old.end() && p->second.specs() == ps.second) parameters_[ps.first] = p->second;
        else parameters_[ps.first] = Tensor(ctx_, ps.second.shape(), ps.second.dtype(), ps.second.is_trainable());
    }
}

void Net::bind_tensors()
{
    size_t ws = 0;
    for(Connection &c : connections_) {
        ws = std::max(ws, c.ws_size);
        c.input_tensors.clear();
        c.output_tensors.clear();
        c.parameters.clear();
        for(std::string const &n : c.input_names) {
            auto p = tensors_.find(n);
            c.input_tensors.push_back(p == tensors_.end() ? Tensor() : p->second);
        }
        for(std::string const &n : c.output_names) {
            auto p = tensors_.find(n);
            c.output_tensors.push_back(p == tensors_.end() ? Tensor() : p->second);
        }
        for(std::string const &n : c.parameter_names) c.parameters.push_back(parameters_.at(n));
    }
    workspace_ = ws > 0 ? Tensor(ctx_, Shape(ws), uint8_data) : Tensor();
    size_t side_ws = 0;
    for(Step const &st : steps_) if(st.fork_at >= 0) side_ws = std::max(side_ws, connections_[st.conn].ws_size);
    side_workspace_ = side_ws > 0 ? Tensor(ctx_, Shape(side_ws), uint8_data) : Tensor();
}

void Net::setup()
{
    ctx_.activate();
    drop_graph();
    build_plan();
    allocate_tensors();
    allocate_parameters();
    bind_tensors();
    is_setup_ = true;
    forwards_since_change_ = 0;
}

void Net::reshape_input(std::string const &name, Shape const &s)
{
    if(std::find(inputs_.begin(), inputs_.end(), name) == inputs_.end()) throw ValidationError("Unknown input tensor " + name);
    TensorSpecs &ts = tensor_specs_.at(name);
    ts = TensorSpecs(s, ts.dtype());
    // a placeholder that carries the new shape until reshape() re-allocates
    tensors_[name] = Tensor(nullptr, 0, s, ts.dtype());
    drop_graph();
    is_setup_ = false;
}

void Net::reshape()
{
    // the input tensors' handles say what the new input shapes are: either reshape_input() was
    // called, or the caller reshaped net.input(i) itself, as with the reference
    for(std::string const &in : inputs_) {
        auto t = tensors_.find(in);
        if(t != tensors_.end()) tensor_specs_[in] = TensorSpecs(t->second.shape(), t->second.dtype());
    }
    for(Connection &c : connections_) {
        std::vector<Shape> in, out;
        for(size_t i = 0; i < c.input_names.size(); i++) {
            in.push_back(tensor_specs_.at(c.input_names[i]).shape());
            c.input_specs[i] = TensorSpecs(in.back(), c.input_specs[i].dtype());
        }
        c.op->reshape(in, out, c.ws_size);
        DLPRIM_CHECK(out.size() == c.output_names.size());
        for(size_t i = 0; i < out.size(); i++) {
            c.output_specs[i] = TensorSpecs(out[i], c.output_specs[i].dtype());
            tensor_specs_[c.output_names[i]] = c.output_specs[i];
        }
    }
    setup();
}

// -------------------------------------------------------------------------------------------- parameters
void Net::copy_parameters_to_device()
{
    ExecutionContext e;
    for(auto &p : parameters_) p.second.to_device(e, false);
    e.finish();
    for(Connection &c : connections_) c.op->parameters_changed();
    drop_graph();
    forwards_since_change_ = 0;
}
void Net::copy_parameters_to_host()
{
    ExecutionContext e;
    for(auto &p : parameters_) p.second.to_host(e, false);
    e.finish();
}

void Net::save_parameters(std::string const &fname)
{
    json::value header;
    json::value &tensors = header["tensors"];
    tensors = json::object();
    size_t start = 0;
    for(auto &pr : parameters_) {
        json::value &spec = tensors[pr.first];
        spec["dtype"] = data_type_to_string(pr.second.dtype());
        json::array dims;
        for(size_t d : pr.second.shape()) dims.push_back(json::value(double(d)));
        spec["shape"] = dims;
        spec["size"] = double(pr.second.memory_size());
        spec["start"] = double(start);
        start += pr.second.memory_size();
    }
    std::string text = header.save();
    unsigned len = unsigned(text.size());
    std::ofstream f(fname, std::fstream::binary);
    f << "DLPW";
    for(int i = 0; i < 4; i++) f << char(0xFF & (len >> (24 - i * 8)));
    f << text;
    for(auto &pr : parameters_) f.write(static_cast<char *>(pr.second.host_data()), pr.second.memory_size());
    f.flush();
    if(!f) throw ValidationError("I/O error in saving to " + fname);
}

void Net::load_parameters(std::istream &f, bool allow_missing)
{
    unsigned char buf[8] = {0};
    f.read(reinterpret_cast<char *>(buf), 8);
    if(!f || memcmp(buf, "DLPW", 4) != 0) throw ValidationError("Invalid File Format");
    unsigned len = 0;
    for(int i = 0; i < 4; i++) len |= unsigned(buf[4 + i]) << ((3 - i) * 8);
    if(len > 64u * 1024 * 1024) throw ValidationError("Header seems to be too big");
    std::string text(len, '\0');
    f.read(&text[0], len);
    if(!f) throw ValidationError("Problem readfing file");
    json::value header;
    char const *b = text.c_str();
    if(!header.load(b, b + len, true)) throw ValidationError("Problem parsing content");
    std::streamoff base = f.tellg();
    json::object const &tensors = header["tensors"].object();
    for(auto &pr : parameters_) {
        auto p = tensors.find(pr.first);
        if(p == tensors.end()) {
            if(allow_missing) continue;
            throw ValidationError("No parameter " + pr.first + " was found");
        }
        std::vector<int> dims = p->second.get<std::vector<int> >("shape");
        DataType dt = string_to_data_type(p->second.get<std::string>("dtype"));
        Shape shape = Shape::from_range(dims.begin(), dims.end());
        if(shape != pr.second.shape() || dt != pr.second.dtype()) throw ValidationError("Tensor shape/type mistmatch for " + pr.first);
        size_t start = p->second.get<size_t>("start"), size = p->second.get<size_t>("size");
        if(size != pr.second.memory_size()) throw ValidationError("Object size mistmatch");
        f.seekg(base + std::streamoff(start));
        f.read(static_cast<char *>(pr.second.host_data()), size);
        if(!f) throw ValidationError("I/O error");
    }
    copy_parameters_to_device();
}
void Net::load_parameters(std::string const &file_name, bool allow_missing)
{
    std::ifstream f(file_name, std::ifstream::binary);
    if(!f) throw ValidationError("Failed to open file " + file_name);
    load_parameters(f, allow_missing);
}

// -------------------------------------------------------------------------------------------- access
Tensor &Net::tensor(std::string const &name)
{
    auto p = tensors_.find(name);
    if(p == tensors_.end()) throw ValidationError("Unknown tensor name:" + name);
    return p->second;
}
Tensor &Net::param(std::string const &name)
{
    auto p = parameters_.find(name);
    if(p == parameters_.end()) throw ValidationError("Unknown parameter name:" + name);
    return p->second;
}
Tensor &Net::input(unsigned id)
{
    if(id >= inputs_.size()) throw ValidationError("Invalid input id");
    return tensor(inputs_[id]);
}
Tensor &Net::output(unsigned id)
{
    if(id >= outputs_.size()) throw ValidationError("Invalid output id");
    return tensor(outputs_[id]);
}

// -------------------------------------------------------------------------------------------- forward
void Net::run_steps(ExecutionContext const &e)
{
    auto run = [&](Step const &st, ExecutionContext const &ex, Tensor &ws) {
        Connection &c = connections_[st.conn];
        ExecGuard g(ex, c.name.c_str());
        if(st.kind == Step::conv_residual) {
            Convolution2D *conv = static_cast<Convolution2D *>(c.op.get());
            conv->forward_fused(c.input_tensors[0], tensors_.at(st.result), c.parameters, ws, tensors_.at(st.residual),
                                st.residual_scale, st.post_activation, ex);
        }
        else
            c.op->forward(c.input_tensors, c.output_tensors, c.parameters, ws, ex);
    };
    // the second stream is used with a real stream and without per-operator timing (which wants one stream's order)
    bool side = e.stream() != nullptr && !e.timing_enabled();
    if(side) {
        size_t wanted = 0;
        for(Step const &st : steps_) if(st.fork_at >= 0) wanted += 2;
        side = wanted > 0;
        if(side && !side_stream_) cuda_check(cudaStreamCreateWithFlags(&side_stream_, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
        while(side && side_events_.size() < wanted) {
            cudaEvent_t ev;
            cuda_check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreateWithFlags");
            side_events_.push_back(ev);
        }
    }
    ExecutionContext side_e(side_stream_);
    for(int k = 0; k < int(steps_.size()); k++) {
        if(side) {
            size_t ev = 0;
            for(Step const &br : steps_) {
                if(br.fork_at < 0) continue;
                if(br.fork_at == k) {
                    // the branch starts when everything before step k is done, on its own stream and workspace
                    cuda_check(cudaEventRecord(side_events_[ev], e.stream()), "cudaEventRecord");
                    cuda_check(cudaStreamWaitEvent(side_stream_, side_events_[ev], 0), "cudaStreamWaitEvent");
                    run(br, side_e, side_workspace_);
                    cuda_check(cudaEventRecord(side_events_[ev + 1], side_stream_), "cudaEventRecord");
                }
                if(br.join_at == k) cuda_check(cudaStreamWaitEvent(e.stream(), side_events_[ev + 1], 0), "cudaStreamWaitEvent");
                ev += 2;
            }
        }
        Step const &st = steps_[k];
        if(side && st.fork_at >= 0) continue;        // ran on the second stream
        run(st, e, workspace_);
    }
}

void Net::drop_graph()
{
    if(graph_exec_) {
        cudaGraphExecDestroy(graph_exec_);
        graph_exec_ = nullptr;
    }
}

void Net::forward(ExecutionContext const &e, bool sync)
{
    if(!is_setup_) throw ValidationError("Net::setup() must be called before forward()");
    ctx_.activate();
    // The first pass after a change runs operator by operator: it is where operators pack their
    // weights.  The second is recorded into a graph, later ones replay it.  The legacy default
    // stream cannot be captured, so it always runs eagerly.
    const bool graph_ok = use_graph_ && !e.timing_enabled() && e.stream() != nullptr;
    if(graph_ok && graph_exec_ && graph_stream_ == e.stream()) {
        cuda_check(cudaGraphLaunch(graph_exec_, e.stream()), "cudaGraphLaunch");
    }
    else if(graph_ok && forwards_since_change_ >= 1) {
        drop_graph();
        cudaGraph_t graph = nullptr;
        cuda_check(cudaStreamBeginCapture(e.stream(), cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
        try {
            run_steps(e);
        }
        catch(...) {
            cudaStreamEndCapture(e.stream(), &graph);
            if(graph) cudaGraphDestroy(graph);
            throw;
        }
        cuda_check(cudaStreamEndCapture(e.stream(), &graph), "cudaStreamEndCapture");
        cudaError_t err = cudaGraphInstantiate(&graph_exec_, graph, 0);
        cudaGraphDestroy(graph);
        cuda_check(err, "cudaGraphInstantiate");
        graph_stream_ = e.stream();
        cuda_check(cudaGraphLaunch(graph_exec_, e.stream()), "cudaGraphLaunch");
    }
    else
        run_steps(e);
    forwards_since_change_++;
    if(sync) e.finish();
}

std::vector<std::string> Net::describe_plan() const
{
    std::vector<std::string> lines;
    for(Step const &st : steps_) {
        Connection const &c = connections_[st.conn];
        std::string line = c.name + " " + c.op->operator_type();
        if(Convolution2D const *conv = dynamic_cast<Convolution2D const *>(c.op.get()))
            line += std::string(" ") + conv->algo() + " " + conv->kernel_name();
        else if(InnerProduct const *ip = dynamic_cast<InnerProduct const *>(c.op.get()))
            line += std::string(" ") + ip->kernel_name();
        if(st.kind == Step::conv_residual)
            line += " +residual(" + st.residual + ")->" + st.result + " absorbs " + connections_[st.fused_conn].name;
        if(st.fork_at >= 0)
            line += " [second stream: from before " + connections_[steps_[st.fork_at].conn].name + " until " +
                    connections_[steps_[st.join_at].conn].name + "]";
        lines.push_back(line);
    }
    return lines;
}

} // namespace dlprim
