// Stand-in for the reference's dl::Model, for compiling its detection post-processors on the host
// (oracle/_ref): only what vision/detect/*.cpp touch - named output tensors.  Test infrastructure.
#pragma once
#include "dl_tensor_base.hpp"
#include <map>
#include <string>

namespace dl {
class Model {
public:
    std::map<std::string, TensorBase *> outputs;
    TensorBase *get_output(const std::string &name)
    {
        auto it = outputs.find(name);
        return it == outputs.end() ? nullptr : it->second;
    }
};
} // namespace dl
