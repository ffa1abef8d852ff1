// Model<T>: the inference-side model interface (upstream dnn/models/model.cuh:17-46): name, layers,
// forward through every Layer<T> in order (dnn/models/model.cu:8-20), parameters, save.
// TrainingModel<T> keeps the train_step entry points of upstream dnn/models/training_model.cuh:30-79 so that
// model classes written against it compile; losses and optimisers are training-side and outside this
// build, so there are no set_loss / set_optimizer members to call.
#pragma once

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "dnn/core/layer.cuh"

namespace dnn {

template <typename T>
class Model {
public:
    explicit Model(bool training_enabled = false) : training_enabled_(training_enabled) {}
    virtual ~Model() = default;

    virtual std::string name() const { return "DefaultNet"; }
    virtual std::vector<BaseLayer*> layers() = 0;  // non-owning, in execution order

    virtual tensor<T> forward(const tensor<T>& input) {
        tensor<T> x = input.clone();
        for (BaseLayer* base : layers()) {
            auto* layer = dynamic_cast<Layer<T>*>(base);
            if (!layer) throw std::runtime_error("Model::forward: layer " + base->name() + " is not a Layer<T>");
            x = layer->forward(x);
        }
        return x;
    }

    T loss() const { return current_loss_; }

    virtual std::vector<tensor<T>*> parameters() {
        std::vector<tensor<T>*> all;
        for (BaseLayer* base : layers())
            if (auto* layer = dynamic_cast<Layer<T>*>(base)) {
                auto p = layer->parameters();
                all.insert(all.end(), p.begin(), p.end());
            }
        return all;
    }

    bool training_enabled() const { return training_enabled_; }
    virtual void save(const std::string& path) const = 0;

protected:
    T current_loss_ = 0;
    bool training_enabled_;
};

template <typename T>
class TrainingModel : public Model<T> {
public:
    explicit TrainingModel(bool training_enabled = false) : Model<T>(training_enabled) {}
    virtual void train_step(const tensor<T>& input, const tensor<T>& target) = 0;
};

}  // namespace dnn
