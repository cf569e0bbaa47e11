// Registry of layer types: a process-wide map from the prototxt `type` string
// to a creator function, filled by static initialisers (REGISTER_LAYER_CLASS /
// REGISTER_LAYER_CREATOR) and read-only afterwards.  Same plugin interface as
// mini-caffe's src/layer_factory.hpp:54-127; an unknown type fails with the
// list of known types, as there (:76-77).
#ifndef MCB200_LAYER_FACTORY_H_
#define MCB200_LAYER_FACTORY_H_

#include <functional>
#include <map>
#include <string>
#include <vector>

#include "caffe.pb.h"
#include "caffe/base.hpp"

namespace caffe {

class Layer;

class LayerRegistry {
 public:
  using Creator = std::function<shared_ptr<Layer>(const LayerParameter&)>;
  using CreatorRegistry = std::map<string, Creator>;

  static CreatorRegistry& Registry() {
    static CreatorRegistry* table = new CreatorRegistry();  // never destroyed: used by static initialisers
    return *table;
  }

  static void AddCreator(const string& type, Creator creator) {
    CreatorRegistry& table = Registry();
    CHECK_EQ(table.count(type), 0u) << "Layer type " << type << " already registered.";
    table[type] = creator;
  }

  static shared_ptr<Layer> CreateLayer(const LayerParameter& param) {
    const string& type = param.type();
    CreatorRegistry& table = Registry();
    CHECK_EQ(table.count(type), 1u) << "Unknown layer type: " << type << " (known types: "
                                    << LayerTypeListString() << ")";
    return table[type](param);
  }

  static vector<string> LayerTypeList() {
    vector<string> types;
    for (const auto& kv : Registry()) types.push_back(kv.first);
    return types;
  }

 private:
  LayerRegistry() = default;
  DISABLE_COPY_AND_ASSIGN(LayerRegistry);

  static string LayerTypeListString() {
    string joined;
    for (const string& t : LayerTypeList()) {
      if (!joined.empty()) joined += ", ";
      joined += t;
    }
    return joined;
  }
};

class LayerRegister {
 public:
  LayerRegister(const string& type, LayerRegistry::Creator creator) { LayerRegistry::AddCreator(type, creator); }
};

#define REGISTER_LAYER_CREATOR(type, creator) static LayerRegister layer_register_##type(#type, creator)

#define REGISTER_LAYER_CLASS(type)                                                \
  static shared_ptr<Layer> Create##type##Layer(const LayerParameter& param) {     \
    return shared_ptr<Layer>(new type##Layer(param));                             \
  }                                                                               \
  REGISTER_LAYER_CREATOR(type, Create##type##Layer)

}  // namespace caffe

#endif  // MCB200_LAYER_FACTORY_H_
