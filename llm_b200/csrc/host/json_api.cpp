// The JSON reader for callers across the C boundary: a document is parsed once and handed over
// as its nodes in document order (a node's children follow it), which is enough to rebuild
// the value on the other side. Configuration files and checkpoint indexes are read this way.
#include <fstream>
#include <sstream>

#include "json.hpp"

using namespace llmh;

namespace {

struct Node {
    int kind;                 // Json::Kind
    std::string key;          // name if the node is a member of an object
    std::string text;         // strings
    long long integer = 0;
    double real = 0.0;
    int children = 0;
};

struct Document {
    std::vector<Node> nodes;
    void add(const std::string& key, const Json& value) {
        Node node;
        node.kind = value.kind;
        node.key = key;
        node.text = value.string;
        node.integer = value.kind == Json::Bool ? (value.boolean ? 1 : 0) : value.integer;
        node.real = value.real;
        node.children = (int)(value.kind == Json::Object ? value.members.size() : value.items.size());
        nodes.push_back(node);
        for (const auto& member : value.members) add(member.first, member.second);
        for (const Json& item : value.items) add("", item);
    }
};

}  // namespace

LLMH_EXPORT int llmh_json_parse(const char* text, long long size, const char* where, void** out) {
    return guarded([&] {
        Json value = JsonReader(text, (size_t)size, where).read();
        Document* document = new Document();
        document->add("", value);
        *out = document;
    });
}
LLMH_EXPORT void llmh_json_free(void* document) { delete static_cast<Document*>(document); }
LLMH_EXPORT int llmh_json_count(void* document) { return (int)static_cast<Document*>(document)->nodes.size(); }
// kind: 0 null, 1 bool, 2 integer, 3 real, 4 string, 5 array, 6 object
LLMH_EXPORT int llmh_json_node(void* document, int index, int* kind, const char** key, const char** text,
                               long long* integer, double* real, int* children) {
    return guarded([&] {
        const Document* d = static_cast<Document*>(document);
        if (index < 0 || index >= (int)d->nodes.size()) throw Failure{LLMH_INVARIANT, "no such JSON node"};
        const Node& node = d->nodes[index];
        *kind = node.kind;
        *key = node.key.c_str();
        *text = node.text.c_str();
        *integer = node.integer;
        *real = node.real;
        *children = node.children;
    });
}
