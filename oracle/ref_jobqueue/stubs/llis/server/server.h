#pragma once
namespace llis { namespace server { class Server; } }
